// W8A8 MoE expert path: router, routing plan, gather + per-token quant,
// SwiGLU re-quant and weighted combine.  The two grouped int8 GEMMs live in
// w8a8_gemm.cu; this file holds the HBM-bound stages around them and the
// entry point that chains them.
//
// Reference semantics: SmoothQuantPackedMoeExperts.forward
// (algorithm/quantization/ptq/smoothquant/source/smoothquant/fake_quant.py:165-191);
// real-int pipeline shape: _run_expert_tile
// (acceleration/runtime_patches/vllm_ascend.patch:2356-2422) =
// routing+quant -> grouped GEMM1 + SwiGLU + re-quant -> grouped GEMM2 -> unpermute.
//
// Layout: routed rows are sorted by expert; every expert's segment starts at
// a multiple of 128 rows, so a 128-row GEMM tile never straddles experts.
#include "common.cuh"
#include "moe_api.cuh"

namespace mp {

constexpr int kTileRows = kMoeTileRows;
constexpr int kMaxExperts = 256;

// softmax(fp32) -> top-k -> renormalise -> fp16, one thread per token
// (algorithm/quantization/qat/flatquant/source/flatquant/model_tools/mixtral_utils.py:330-333,349).
__global__ void moe_router_topk_kernel(const float* __restrict__ logits, int T, int E, int k,
                                       int* __restrict__ idx, __half* __restrict__ w) {
  const int t = blockIdx.x * blockDim.x + threadIdx.x;
  if (t >= T) return;
  const float* l = logits + (size_t)t * E;
  float mx = -INFINITY;
  for (int e = 0; e < E; ++e) mx = fmaxf(mx, l[e]);
  float sum = 0.0f;
  for (int e = 0; e < E; ++e) sum += expf(l[e] - mx);
  float chosen_p[8];
  int chosen[8];
  float psum = 0.0f;
  for (int j = 0; j < k; ++j) {
    float best = -1.0f;
    int bi = 0;
    for (int e = 0; e < E; ++e) {
      bool taken = false;
      for (int i = 0; i < j; ++i) taken |= (chosen[i] == e);
      const float pe = expf(l[e] - mx) / sum;
      if (!taken && pe > best) { best = pe; bi = e; }     // strict >: ties go to the lower index
    }
    chosen[j] = bi;
    chosen_p[j] = best;
    psum += best;
  }
  for (int j = 0; j < k; ++j) {
    idx[(size_t)t * k + j] = chosen[j];
    w[(size_t)t * k + j] = f2h(chosen_p[j] / psum);
  }
}

// counts[e] = routed entries whose expert is local expert e (experts [lo, hi)).
__global__ void moe_count_kernel(const int* __restrict__ ids, int n_entries, int lo, int hi, int* __restrict__ counts) {
  __shared__ int s_counts[kMaxExperts];
  for (int i = threadIdx.x; i < hi - lo; i += blockDim.x) s_counts[i] = 0;
  __syncthreads();
  for (int i = blockIdx.x * blockDim.x + threadIdx.x; i < n_entries; i += gridDim.x * blockDim.x) {
    const int e = ids[i];
    if (e >= lo && e < hi) atomicAdd(&s_counts[e - lo], 1);
  }
  __syncthreads();
  for (int i = threadIdx.x; i < hi - lo; i += blockDim.x)
    if (s_counts[i]) atomicAdd(&counts[i], s_counts[i]);
}

// Padded segment offsets (multiples of 256 rows), the expert of every 128-row tile and the tile count.
// plan layout (ints): [0,E) counts | [E,2E) cursors | [2E,3E+1) seg_offsets | 3E+1 num_tiles | 3E+2.. tile_expert
__global__ void moe_plan_kernel(int* __restrict__ plan, int E, int max_tiles) {
  if (threadIdx.x != 0 || blockIdx.x != 0) return;
  int* counts = plan;
  int* cursors = plan + E;
  int* seg = plan + 2 * E;
  int* num_tiles = plan + 3 * E + 1;
  int* tile_expert = plan + 3 * E + 2;
  int off = 0, tiles = 0;
  for (int e = 0; e < E; ++e) {
    seg[e] = off;
    cursors[e] = 0;
    const int nt = moe_segment_tiles(counts[e]);
    for (int i = 0; i < nt && tiles < max_tiles; ++i) tile_expert[tiles++] = e;
    off += nt * kTileRows;
  }
  seg[E] = off;
  *num_tiles = tiles;
}

// Count and plan in one launch (one block): the per-expert counts are taken in shared memory, thread 0 lays out the
// padded segments exactly as moe_plan_kernel does, and the scales of every segment's padding rows are zeroed -- so
// the routing needs no memset of the counters or of the scale buffer and two launches instead of five nodes.
__global__ void __launch_bounds__(1024)
moe_count_plan_kernel(const int* __restrict__ ids, int n_entries, int lo, int hi, int* __restrict__ plan, int E,
                      int max_tiles, float* __restrict__ routed_scale) {
  chain_wait();
  chain_release();
  __shared__ int s_counts[kMaxExperts];
  for (int i = threadIdx.x; i < E; i += blockDim.x) s_counts[i] = 0;
  __syncthreads();
  for (int i0 = 0; i0 < n_entries; i0 += blockDim.x) {          // uniform trip count: the vote below is warp-wide
    const int i = i0 + threadIdx.x;
    const int e = i < n_entries ? ids[i] : -1;
    const int key = (e >= lo && e < hi) ? e - lo : -1;
    const unsigned int same = __match_any_sync(0xffffffffu, key);   // one shared-memory add per expert and warp
    if (key >= 0 && (threadIdx.x & 31) == __ffs(same) - 1) atomicAdd(&s_counts[key], __popc(same));
  }
  __syncthreads();
  int* counts = plan;
  int* cursors = plan + E;
  int* seg = plan + 2 * E;
  if (threadIdx.x == 0) {
    int* num_tiles = plan + 3 * E + 1;
    int* tile_expert = plan + 3 * E + 2;
    int off = 0, tiles = 0;
    for (int e = 0; e < E; ++e) {
      counts[e] = s_counts[e];
      seg[e] = off;
      cursors[e] = 0;
      const int nt = moe_segment_tiles(s_counts[e]);
      for (int i = 0; i < nt && tiles < max_tiles; ++i) tile_expert[tiles++] = e;
      off += nt * kTileRows;
    }
    seg[E] = off;
    *num_tiles = tiles;
  }
  __syncthreads();
  // padding rows get scale 0, so whatever codes they hold turn into zeros downstream
  for (int e = 0; e < E; ++e)
    for (int r = seg[e] + s_counts[e] + threadIdx.x; r < seg[e + 1]; r += blockDim.x) routed_scale[r] = 0.0f;
  for (int r = seg[E] + threadIdx.x; r < max_tiles * kTileRows; r += blockDim.x) routed_scale[r] = 0.0f;   // unused tail
}

// One block per routed entry (t, j): claim a row in the expert's segment, record it, and
// write the token's int8 codes and scale there -- the gather and the per-token quant of
// npu_moe_init_routing_quant (acceleration/runtime_patches/vllm_ascend.patch:2369-2379)
// in one pass.  Arithmetic as in act_quant.cu.
// KEEP: rows of up to 4096 values (two 16-byte pieces per thread) stay in registers between the abs-max pass
// and the quantising pass instead of being read a second time.
template <bool KEEP>
__global__ void __launch_bounds__(256)
moe_gather_quant_kernel(const __half* __restrict__ hidden, const int* __restrict__ ids, int H, int k, int lo, int hi,
                        int* __restrict__ plan, int E, int* __restrict__ dest_row,
                        int8_t* __restrict__ routed_q, float* __restrict__ routed_scale) {
  chain_wait();
  chain_release();
  __shared__ float s_red[8];
  __shared__ float s_scale;
  __shared__ int s_dest;
  const int entry = blockIdx.x;
  const int e = ids[entry];
  if (e < lo || e >= hi) {
    if (threadIdx.x == 0) dest_row[entry] = -1;
    return;
  }
  const int t = entry / k;
  const __half* xr = hidden + (size_t)t * H;
  const int chunks = H >> 3;
  float amax = 0.0f;
  [[maybe_unused]] uint4 kept[2];
  if constexpr (KEEP) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = threadIdx.x + 256 * i;
      kept[i] = c < chunks ? *reinterpret_cast<const uint4*>(xr + c * 8) : make_uint4(0, 0, 0, 0);
      const __half2* h2 = reinterpret_cast<const __half2*>(&kept[i]);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __half22float2(__habs2(h2[j]));
        amax = fmaxf(amax, fmaxf(f.x, f.y));
      }
    }
  } else {
    for (int c = threadIdx.x; c < chunks; c += 256) {
      uint4 raw = *reinterpret_cast<const uint4*>(xr + c * 8);
      const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
      for (int j = 0; j < 4; ++j) {
        float2 f = __half22float2(__habs2(h2[j]));
        amax = fmaxf(amax, fmaxf(f.x, f.y));
      }
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x == 0) {
    float v = s_red[0];
#pragma unroll
    for (int i = 1; i < 8; ++i) v = fmaxf(v, s_red[i]);
    const float eps = h2f(f2h(1e-5f));
    s_scale = h2f(f2h(__fdiv_rn(fmaxf(v, eps), 127.0f)));
    const int pos = atomicAdd(plan + E + (e - lo), 1);
    s_dest = plan[2 * E + (e - lo)] + pos;
    dest_row[entry] = s_dest;
    routed_scale[s_dest] = s_scale;
  }
  __syncthreads();
  const float sf = s_scale;
  const RowQuant rq = make_row_quant(sf);
  int8_t* qr = routed_q + (size_t)s_dest * H;
  if constexpr (KEEP) {
#pragma unroll
    for (int i = 0; i < 2; ++i) {
      const int c = threadIdx.x + 256 * i;
      if (c < chunks) *reinterpret_cast<uint2*>(qr + c * 8) = quant8_pack(kept[i], rq);
    }
  } else {
    for (int c = threadIdx.x; c < chunks; c += 256) {
      uint4 raw = *reinterpret_cast<const uint4*>(xr + c * 8);
      *reinterpret_cast<uint2*>(qr + c * 8) = quant8_pack(raw, rq);
    }
  }
}

// Second activation quant (fake_quant.py:186) with the abs-max of every row within every 128-column tile already
// known from the GEMM1 epilogue (absmax[row][slots]): the row's maximum is the maximum of its slots, then one pass
// over h.
__global__ void __launch_bounds__(256)
moe_requant_kernel(const __half* __restrict__ h, const float* __restrict__ absmax, int slots, int I,
                   const int* __restrict__ num_tiles, int8_t* __restrict__ q, float* __restrict__ scale) {
  chain_wait();
  chain_release();
  constexpr int kBatch = 32;                                     // rows whose scales are found before they stream
  __shared__ float s_scale[kBatch];
  const int rows = *num_tiles * kTileRows;                       // rows in use; the grid strides over them
  const float eps = h2f(f2h(1e-5f));
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  for (int row0 = blockIdx.x; row0 < rows; row0 += gridDim.x * kBatch) {
    // a warp per row: the maximum of the row's slots, then the scale
    for (int i = warp; i < kBatch; i += 8) {
      const int row = row0 + i * gridDim.x;
      if (row >= rows) break;
      float m = 0.0f;
      for (int j = lane; j < slots; j += 32) m = fmaxf(m, absmax[(size_t)row * slots + j]);
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
      if (lane == 0) {
        const float sf = h2f(f2h(__fdiv_rn(fmaxf(m, eps), 127.0f)));
        s_scale[i] = sf;
        scale[row] = sf;
      }
    }
    __syncthreads();
    for (int i = 0; i < kBatch; ++i) {
      const int row = row0 + i * gridDim.x;
      if (row >= rows) break;
      const RowQuant rq = make_row_quant(s_scale[i]);
      const __half* hr = h + (size_t)row * I;
      int8_t* qr = q + (size_t)row * I;
      for (int c = threadIdx.x; c < (I >> 3); c += 256) {
        uint4 raw = *reinterpret_cast<const uint4*>(hr + c * 8);
        *reinterpret_cast<uint2*>(qr + c * 8) = quant8_pack(raw, rq);
      }
    }
    __syncthreads();                                              // s_scale is rewritten by the next batch
  }
}

static int launch_requant(const __half* h, const float* absmax, int I, const int* num_tiles, int padded_rows,
                          int8_t* q2, float* scale2, cudaStream_t st) {
  const int grid = padded_rows < 8 * kSmCount ? padded_rows : 8 * kSmCount;
  return launch_chained(moe_requant_kernel, dim3(grid), dim3(256), 0, st, h, absmax, moe_absmax_slots(I), I, num_tiles,
                        q2, scale2);
}

// out[t] = sum_j f16(d[dest(t,j)] * w[t,j]) with fp16 adds, visiting the token's experts in
// ascending order as the reference's per-expert index_add_ does (fake_quant.py:188-189).
// Entries routed elsewhere (dest < 0) contribute nothing.
// Expert-parallel form (arrivals != null): the rows of d are stored by the peers, each of which then raises its
// arrival word here (arrivals[r], see the push kernel in moe_ep.cu) to the epoch this rank's own push has just
// written to *epoch; every block waits for all of them (bounded) before it reads a row.
__global__ void __launch_bounds__(256)
moe_combine_kernel(const __half* __restrict__ d, const int* __restrict__ dest_row, const int* __restrict__ ids,
                   const __half* __restrict__ weights, int T, int H, int k, __half* __restrict__ out,
                   const unsigned int* arrivals, int world, const unsigned int* epoch, int* error_word) {
  chain_wait();
  chain_release();
  if (arrivals != nullptr) {
    if (static_cast<int>(threadIdx.x) < world) {
      peer_flag_wait(arrivals + threadIdx.x, *epoch, error_word);
      __threadfence_system();
    }
    __syncthreads();
  }
  const int t = blockIdx.x;
  int order[8];
  for (int j = 0; j < k; ++j) order[j] = j;
  for (int a = 1; a < k; ++a)                      // insertion sort by expert id (k is tiny)
    for (int b = a; b > 0 && ids[(size_t)t * k + order[b]] < ids[(size_t)t * k + order[b - 1]]; --b) {
      const int tmp = order[b]; order[b] = order[b - 1]; order[b - 1] = tmp;
    }
  for (int c = threadIdx.x; c < (H >> 3); c += 256) {
    __half acc[8];
#pragma unroll
    for (int i = 0; i < 8; ++i) acc[i] = f2h(0.0f);
    for (int jj = 0; jj < k; ++jj) {
      const int j = order[jj];
      const int r = dest_row[(size_t)t * k + j];
      if (r < 0) continue;
      const __half wj = weights[(size_t)t * k + j];
      uint4 raw = *reinterpret_cast<const uint4*>(d + (size_t)r * H + c * 8);
      const __half* v = reinterpret_cast<const __half*>(&raw);
#pragma unroll
      for (int i = 0; i < 8; ++i) acc[i] = hadd_t(acc[i], hmul_t(v[i], wj));
    }
    *reinterpret_cast<uint4*>(out + (size_t)t * H + c * 8) = *reinterpret_cast<uint4*>(acc);
  }
}

// dst row i = src row map[i] (16-byte vectors); map[i] < 0 leaves zeros.  Used to compact
// the rows an expert-parallel rank receives from its peers into expert-sorted order, and back.
__global__ void __launch_bounds__(256)
gather_rows_kernel(const uint4* __restrict__ src, const int* __restrict__ map, int vec_per_row,
                   uint4* __restrict__ dst) {
  const int row = blockIdx.x;
  const int s = map[row];
  for (int v = threadIdx.x; v < vec_per_row; v += 256)
    dst[(size_t)row * vec_per_row + v] = s >= 0 ? src[(size_t)s * vec_per_row + v] : make_uint4(0, 0, 0, 0);
}

__global__ void gather_words_kernel(const uint32_t* __restrict__ src, const int* __restrict__ map, int n,
                                    uint32_t* __restrict__ dst) {
  const int i = blockIdx.x * blockDim.x + threadIdx.x;
  if (i < n) dst[i] = map[i] >= 0 ? src[map[i]] : 0u;
}

}  // namespace mp

using namespace mp;

extern "C" int mp_gather_rows(const void* src, const void* row_map_i32, int n_dst_rows, int row_bytes, void* dst,
                              mp_stream_t stream) {
  if (!src || !row_map_i32 || !dst || n_dst_rows < 0 || row_bytes <= 0) return MP_ERR_INVALID_ARG;
  if (n_dst_rows == 0) return MP_OK;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  if (row_bytes == 4) {
    gather_words_kernel<<<(n_dst_rows + 255) / 256, 256, 0, st>>>(
        static_cast<const uint32_t*>(src), static_cast<const int*>(row_map_i32), n_dst_rows, static_cast<uint32_t*>(dst));
  } else {
    if (row_bytes % 16 != 0) return MP_ERR_UNSUPPORTED;
    if (!aligned(src, 16) || !aligned(dst, 16)) return MP_ERR_ALIGNMENT;
    gather_rows_kernel<<<n_dst_rows, 256, 0, st>>>(static_cast<const uint4*>(src), static_cast<const int*>(row_map_i32),
                                                   row_bytes / 16, static_cast<uint4*>(dst));
  }
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" int mp_moe_router_topk(const void* logits_f32, int T, int E, int k, void* idx_i32, void* weights_f16,
                                  mp_stream_t stream) {
  if (!logits_f32 || !idx_i32 || !weights_f16 || T <= 0 || E <= 0 || k <= 0) return MP_ERR_INVALID_ARG;
  if (k > 8 || k > E) return MP_ERR_UNSUPPORTED;
  moe_router_topk_kernel<<<(T + 127) / 128, 128, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const float*>(logits_f32), T, E, k, static_cast<int*>(idx_i32), static_cast<__half*>(weights_f16));
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" size_t mp_moe_plan_ints(int num_local_experts, int max_rows) {
  const int max_tiles = mp_moe_padded_rows(num_local_experts, max_rows) / kTileRows;
  return (size_t)3 * num_local_experts + 2 + max_tiles;
}

extern "C" int mp_moe_padded_rows(int num_local_experts, int max_rows) {
  return (max_rows / kMoeSegmentAlign + num_local_experts) * kMoeSegmentAlign;
}

extern "C" int mp_moe_route_gather_quant(const void* hidden_f16, const void* topk_ids_i32, int T, int H, int k,
                                         int expert_lo, int expert_hi, void* plan_i32, void* dest_row_i32,
                                         void* routed_q_i8, void* routed_scale_f32, mp_stream_t stream) {
  if (!hidden_f16 || !topk_ids_i32 || !plan_i32 || !dest_row_i32 || !routed_q_i8 || !routed_scale_f32 || T <= 0 ||
      H <= 0 || k <= 0)
    return MP_ERR_INVALID_ARG;
  const int E = expert_hi - expert_lo;
  if (E <= 0 || E > kMaxExperts || H % 16 != 0 || k > 8) return MP_ERR_UNSUPPORTED;
  if (!aligned(hidden_f16, 16) || !aligned(routed_q_i8, 16)) return MP_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  int* plan = static_cast<int*>(plan_i32);
  const int n_entries = T * k;
  const int padded = mp_moe_padded_rows(E, n_entries);
  if (n_entries <= 8192) {
    // few entries (a rank's share under expert parallelism, decode batches): one block counts, plans and zeroes the
    // padding rows' scales -- two launches instead of five graph nodes; with more entries one block's pass over the
    // ids costs what the extra nodes do (16384 entries: equal within 0.2 %), so those keep the multi-block count
    const int rc = launch_chained(moe_count_plan_kernel, dim3(1), dim3(1024), 0, st,
                                  static_cast<const int*>(topk_ids_i32), n_entries, expert_lo, expert_hi, plan, E,
                                  padded / kTileRows, static_cast<float*>(routed_scale_f32));
    if (rc != MP_OK) return rc;
  } else {
    MP_CUDA_TRY(cudaMemsetAsync(plan, 0, sizeof(int) * E, st));
    // padding rows get scale 0, so whatever codes they hold turn into zeros downstream
    MP_CUDA_TRY(cudaMemsetAsync(routed_scale_f32, 0, sizeof(float) * padded, st));
    int blocks = (n_entries + 255) / 256;
    if (blocks > 4 * kSmCount) blocks = 4 * kSmCount;
    moe_count_kernel<<<blocks, 256, 0, st>>>(static_cast<const int*>(topk_ids_i32), n_entries, expert_lo, expert_hi, plan);
    MP_LAUNCH_CHECK();
    moe_plan_kernel<<<1, 32, 0, st>>>(plan, E, padded / kTileRows);
    MP_LAUNCH_CHECK();
  }
  return launch_chained(H <= 4096 ? moe_gather_quant_kernel<true> : moe_gather_quant_kernel<false>, dim3(n_entries),
                        dim3(256), 0, st,
                        static_cast<const __half*>(hidden_f16), static_cast<const int*>(topk_ids_i32), H, k, expert_lo,
                        expert_hi, plan, E, static_cast<int*>(dest_row_i32), static_cast<int8_t*>(routed_q_i8),
                        static_cast<float*>(routed_scale_f32));
}

// ---- expert stage on rows that are already routed and quantised ------------
// Workspace (bytes, each part 256-byte aligned):
//   h f16 [P, I] | absmax f32 [P, ceil(I / 128)] | q2 i8 [P, I] | scale2 f32 [P]
static size_t align256(size_t x) { return (x + 255) & ~size_t(255); }

extern "C" size_t mp_moe_expert_stage_workspace_bytes(int padded_rows, int I) {
  if (padded_rows <= 0 || I <= 0) return 0;
  const size_t P = (size_t)padded_rows;
  return align256(P * I * 2) + align256(P * moe_absmax_slots(I) * 4) + align256(P * I) + align256(P * 4);
}

struct StageBuffers {
  __half* h;
  float* absmax;
  int8_t* q2;
  float* scale2;
};
static int stage_buffers(void* workspace, size_t workspace_bytes, int padded_rows, int I, StageBuffers& b) {
  if (padded_rows <= 0 || I <= 0) return MP_ERR_INVALID_ARG;
  if (padded_rows % kMoeSegmentAlign != 0 || I % 16 != 0) return MP_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < mp_moe_expert_stage_workspace_bytes(padded_rows, I)) return MP_ERR_WORKSPACE;
  if (!aligned(workspace, 256)) return MP_ERR_ALIGNMENT;
  const size_t P = (size_t)padded_rows;
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  b.h = reinterpret_cast<__half*>(ws);
  ws += align256(P * I * 2);
  b.absmax = reinterpret_cast<float*>(ws);
  ws += align256(P * moe_absmax_slots(I) * 4);
  b.q2 = reinterpret_cast<int8_t*>(ws);
  ws += align256(P * I);
  b.scale2 = reinterpret_cast<float*>(ws);
  return MP_OK;
}

static int expert_stage(const void* routed_q_i8, const void* routed_scale_f32, const void* plan_i32, int padded_rows,
                        int H, int I, int num_local_experts, const void* w13_q_i8, const void* w13_scale_f32,
                        const void* w2_q_i8, const void* w2_scale_f32, void* d_out_f16, const RowScatter* scatter,
                        void* workspace, size_t workspace_bytes, int* error_word, mp_stream_t stream) {
  if (!routed_q_i8 || !routed_scale_f32 || !plan_i32 || !w13_q_i8 || !w13_scale_f32 || !w2_q_i8 || !w2_scale_f32 ||
      (!d_out_f16 && !scatter) || padded_rows <= 0 || H <= 0 || I <= 0 || num_local_experts <= 0)
    return MP_ERR_INVALID_ARG;
  if (H % 16 != 0 || num_local_experts > kMaxExperts) return MP_ERR_UNSUPPORTED;
  StageBuffers b;
  int rc = stage_buffers(workspace, workspace_bytes, padded_rows, I, b);
  if (rc != MP_OK) return rc;
  if (!aligned(routed_q_i8, 16) || !aligned(w13_q_i8, 16) || !aligned(w2_q_i8, 16) ||
      (d_out_f16 && !aligned(d_out_f16, 16)))
    return MP_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int E = num_local_experts;
  const int* plan = static_cast<const int*>(plan_i32);
  const int* num_tiles = plan + 3 * E + 1;
  const int* tile_expert = plan + 3 * E + 2;
  rc = launch_moe_gemm1_swiglu(routed_q_i8, static_cast<const float*>(routed_scale_f32), w13_q_i8,
                               static_cast<const float*>(w13_scale_f32), padded_rows, H, I, E, num_tiles, tile_expert,
                               b.h, b.absmax, error_word, st);
  if (rc != MP_OK) return rc;
  rc = launch_requant(b.h, b.absmax, I, num_tiles, padded_rows, b.q2, b.scale2, st);
  if (rc != MP_OK) return rc;
  return launch_moe_gemm2(b.q2, b.scale2, w2_q_i8, static_cast<const float*>(w2_scale_f32), padded_rows, I, H, E,
                          num_tiles, tile_expert, d_out_f16, error_word, st, scatter);
}

// ---- the expert stage in three launches, each GEMM optionally on one half of the row tiles -----------------
// Same workspace layout and arithmetic as mp_moe_expert_stage; a caller that overlaps the exchange with the GEMMs
// runs: gemm1(half 0) | gemm1(half 1) | requant | gemm2(half 0) | gemm2(half 1), with the pull of half 1 next to
// gemm1(half 0) and the push of half 0 next to gemm2(half 1) on a second stream.
extern "C" int mp_moe_gemm1_swiglu(const void* routed_q_i8, const void* routed_scale_f32, const void* plan_i32,
                                   int padded_rows, int H, int I, int num_local_experts, const void* w13_q_i8,
                                   const void* w13_scale_f32, void* workspace, size_t workspace_bytes, int tile_part,
                                   int* error_word, mp_stream_t stream) {
  if (!routed_q_i8 || !routed_scale_f32 || !plan_i32 || !w13_q_i8 || !w13_scale_f32 || H <= 0 || num_local_experts <= 0 ||
      tile_part < -1 || tile_part > 1)
    return MP_ERR_INVALID_ARG;
  if (H % 16 != 0 || num_local_experts > kMaxExperts) return MP_ERR_UNSUPPORTED;
  if (!aligned(routed_q_i8, 16) || !aligned(w13_q_i8, 16)) return MP_ERR_ALIGNMENT;
  StageBuffers b;
  const int rc = stage_buffers(workspace, workspace_bytes, padded_rows, I, b);
  if (rc != MP_OK) return rc;
  const int E = num_local_experts;
  const int* plan = static_cast<const int*>(plan_i32);
  return launch_moe_gemm1_swiglu(routed_q_i8, static_cast<const float*>(routed_scale_f32), w13_q_i8,
                                 static_cast<const float*>(w13_scale_f32), padded_rows, H, I, E, plan + 3 * E + 1,
                                 plan + 3 * E + 2, b.h, b.absmax, error_word, static_cast<cudaStream_t>(stream), tile_part);
}

extern "C" int mp_moe_requant(const void* plan_i32, int padded_rows, int I, int num_local_experts, void* workspace,
                              size_t workspace_bytes, mp_stream_t stream) {
  if (!plan_i32 || num_local_experts <= 0 || num_local_experts > kMaxExperts) return MP_ERR_INVALID_ARG;
  StageBuffers b;
  const int rc = stage_buffers(workspace, workspace_bytes, padded_rows, I, b);
  if (rc != MP_OK) return rc;
  const int* plan = static_cast<const int*>(plan_i32);
  return launch_requant(b.h, b.absmax, I, plan + 3 * num_local_experts + 1, padded_rows, b.q2, b.scale2,
                        static_cast<cudaStream_t>(stream));
}

extern "C" int mp_moe_gemm2(const void* plan_i32, int padded_rows, int I, int H, int num_local_experts,
                            const void* w2_q_i8, const void* w2_scale_f32, void* d_out_f16, void* workspace,
                            size_t workspace_bytes, int tile_part, int* error_word, mp_stream_t stream) {
  if (!plan_i32 || !w2_q_i8 || !w2_scale_f32 || !d_out_f16 || H <= 0 || num_local_experts <= 0 || tile_part < -1 ||
      tile_part > 1)
    return MP_ERR_INVALID_ARG;
  if (H % 16 != 0 || num_local_experts > kMaxExperts) return MP_ERR_UNSUPPORTED;
  if (!aligned(w2_q_i8, 16) || !aligned(d_out_f16, 16)) return MP_ERR_ALIGNMENT;
  StageBuffers b;
  const int rc = stage_buffers(workspace, workspace_bytes, padded_rows, I, b);
  if (rc != MP_OK) return rc;
  const int E = num_local_experts;
  const int* plan = static_cast<const int*>(plan_i32);
  return launch_moe_gemm2(b.q2, b.scale2, w2_q_i8, static_cast<const float*>(w2_scale_f32), padded_rows, I, H, E,
                          plan + 3 * E + 1, plan + 3 * E + 2, d_out_f16, error_word, static_cast<cudaStream_t>(stream),
                          nullptr, tile_part);
}

extern "C" int mp_moe_expert_stage(const void* routed_q_i8, const void* routed_scale_f32, const void* plan_i32,
                                   int padded_rows, int H, int I, int num_local_experts,
                                   const void* w13_q_i8, const void* w13_scale_f32, const void* w2_q_i8,
                                   const void* w2_scale_f32, void* d_out_f16, void* workspace,
                                   size_t workspace_bytes, int* error_word, mp_stream_t stream) {
  return expert_stage(routed_q_i8, routed_scale_f32, plan_i32, padded_rows, H, I, num_local_experts, w13_q_i8,
                      w13_scale_f32, w2_q_i8, w2_scale_f32, d_out_f16, nullptr, workspace, workspace_bytes, error_word,
                      stream);
}

// Expert-parallel form: the second GEMM's epilogue stores every result row straight into the result buffer
// of the rank the token came from (peer stores over NVLink, located through the extended plan), so no
// sorted result buffer and no separate return kernel exist.  xplan_i32 is the plan mp_moe_ep_plan wrote
// (it begins with the standard plan); capacity_rows as given there.
extern "C" int mp_moe_expert_stage_scatter(const void* routed_q_i8, const void* routed_scale_f32, const void* xplan_i32,
                                           int capacity_rows, int H, int I, int num_local_experts, int world,
                                           const void* w13_q_i8, const void* w13_scale_f32, const void* w2_q_i8,
                                           const void* w2_scale_f32, void* const* peer_back_ptrs, void* workspace,
                                           size_t workspace_bytes, int* error_word, mp_stream_t stream) {
  if (!peer_back_ptrs || world < 1 || world > kMoeMaxRanks || !xplan_i32) return MP_ERR_INVALID_ARG;
  RowScatter sc{};
  sc.xplan = static_cast<const int*>(xplan_i32);
  sc.world = world;
  sc.e_loc = num_local_experts;
  sc.ext = 3 * num_local_experts + 2 + capacity_rows / kTileRows;
  for (int r = 0; r < world; ++r) {
    if (!peer_back_ptrs[r]) return MP_ERR_INVALID_ARG;
    if (!aligned(peer_back_ptrs[r], 16)) return MP_ERR_ALIGNMENT;
    sc.back[r] = peer_back_ptrs[r];
  }
  return expert_stage(routed_q_i8, routed_scale_f32, xplan_i32, capacity_rows, H, I, num_local_experts, w13_q_i8,
                      w13_scale_f32, w2_q_i8, w2_scale_f32, nullptr, &sc, workspace, workspace_bytes, error_word,
                      stream);
}

extern "C" int mp_moe_combine(const void* d_f16, const void* dest_row_i32, const void* topk_ids_i32,
                              const void* topk_weights_f16, int T, int H, int k, void* out_f16, mp_stream_t stream) {
  if (!d_f16 || !dest_row_i32 || !topk_ids_i32 || !topk_weights_f16 || !out_f16 || T <= 0 || H <= 0 || k <= 0)
    return MP_ERR_INVALID_ARG;
  if (H % 8 != 0 || k > 8) return MP_ERR_UNSUPPORTED;
  if (!aligned(d_f16, 16) || !aligned(out_f16, 16)) return MP_ERR_ALIGNMENT;
  return launch_chained(moe_combine_kernel, dim3(T), dim3(256), 0, static_cast<cudaStream_t>(stream),
                        static_cast<const __half*>(d_f16), static_cast<const int*>(dest_row_i32),
                        static_cast<const int*>(topk_ids_i32), static_cast<const __half*>(topk_weights_f16), T, H, k,
                        static_cast<__half*>(out_f16), static_cast<const unsigned int*>(nullptr), 0,
                        static_cast<const unsigned int*>(nullptr), static_cast<int*>(nullptr));
}

extern "C" int mp_moe_combine_after_peers(const void* arrival_words_u32, int world, const void* epoch_counter_u32,
                                          const void* d_f16, const void* dest_row_i32, const void* topk_ids_i32,
                                          const void* topk_weights_f16, int T, int H, int k, void* out_f16,
                                          int* error_word, mp_stream_t stream) {
  if (!arrival_words_u32 || !epoch_counter_u32 || world <= 0 || world > kMoeMaxRanks || !d_f16 || !dest_row_i32 ||
      !topk_ids_i32 || !topk_weights_f16 || !out_f16 || T <= 0 || H <= 0 || k <= 0)
    return MP_ERR_INVALID_ARG;
  if (H % 8 != 0 || k > 8) return MP_ERR_UNSUPPORTED;
  if (!aligned(d_f16, 16) || !aligned(out_f16, 16)) return MP_ERR_ALIGNMENT;
  return launch_chained(moe_combine_kernel, dim3(T), dim3(256), 0, static_cast<cudaStream_t>(stream),
                        static_cast<const __half*>(d_f16), static_cast<const int*>(dest_row_i32),
                        static_cast<const int*>(topk_ids_i32), static_cast<const __half*>(topk_weights_f16), T, H, k,
                        static_cast<__half*>(out_f16), static_cast<const unsigned int*>(arrival_words_u32), world,
                        static_cast<const unsigned int*>(epoch_counter_u32), error_word);
}
