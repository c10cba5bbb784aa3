// Dense chunked gate/up projection with SwiGLU and per-token re-quantisation on int8 rows:
//   for every chunk c:  h_c = silu(x W_gate_c^T) * (x W_up_c^T),  (q_c, s_c) = per-token int8 quant of h_c.
//
// The role of the reference's native op grouped_swiglu_loop_out
// (acceleration/custom_ops/qwen2_5_vl/aclnn_grouped_swiglu_out_bridge.cpp:157-273): one
// grouped-matmul + SwiGLU + quant call per intermediate chunk, every call over the same int8 rows,
// results written into slices of one [chunks, T, C] code tensor and one [chunks, T] scale tensor.  Here
// the chunks are the groups of ONE launch of the grouped tcgen05 int8 GEMM with the SwiGLU epilogue
// (w8a8_gemm.cu), so a short batch still fills the GPU: the rows are replicated once per chunk into
// 256-row aligned segments (the form the reference's own "batched_repeat" route for short batches takes,
// acceleration/runtime_patches/vllm.patch:139-160), the GEMM writes h and each row's max |h|, and one
// pass turns h into codes at the rows' final places.
#include "common.cuh"
#include "moe_api.cuh"

namespace mp {

// Replicate the rows (16 bytes per thread) and write the tile plan.  Rows [T, t_pad) of every segment
// get scale 0: whatever codes they hold turn into zeros in the epilogue, and they are never stored.
__global__ void __launch_bounds__(256)
chunk_stage_kernel(const uint4* __restrict__ x, const float* __restrict__ x_scale, int T, int t_pad, int vec_per_row,
                   int chunks, uint4* __restrict__ x_rep, float* __restrict__ scale_rep, int* __restrict__ plan) {
  chain_wait();                                     // programmatic dependent launch: the producer of x has finished
  chain_release();
  const int row = blockIdx.x;                       // row of the replicated buffer
  const int t = row % t_pad;
  if (row == 0) {
    const int tiles_per_chunk = t_pad / kMoeTileRows;
    for (int i = threadIdx.x; i < chunks * tiles_per_chunk; i += 256) plan[1 + i] = i / tiles_per_chunk;
    if (threadIdx.x == 0) plan[0] = chunks * tiles_per_chunk;
  }
  if (t >= T) {
    if (threadIdx.x == 0) scale_rep[row] = 0.0f;
    return;
  }
  if (threadIdx.x == 0) scale_rep[row] = x_scale[t];
  const uint4* src = x + (size_t)t * vec_per_row;
  uint4* dst = x_rep + (size_t)row * vec_per_row;
  for (int v = threadIdx.x; v < vec_per_row; v += 256) dst[v] = __ldg(src + v);
}

// Per-token quantisation of h with the maxima the GEMM epilogue already found (one per row and 128-column tile);
// arithmetic of the second activation quant in the expert path (moe.cu), rows written to out[c, t, :].
__global__ void __launch_bounds__(256)
chunk_requant_kernel(const __half* __restrict__ h, const float* __restrict__ absmax, int slots, int T, int t_pad,
                     int C, int8_t* __restrict__ q, float* __restrict__ scale) {
  chain_wait();
  chain_release();
  __shared__ float s_red[8];
  const int c = blockIdx.x / T, t = blockIdx.x % T;
  const size_t src_row = (size_t)c * t_pad + t;
  float m = 0.0f;
  for (int i = threadIdx.x; i < slots; i += 256) m = fmaxf(m, absmax[src_row * slots + i]);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) m = fmaxf(m, __shfl_xor_sync(0xffffffffu, m, o));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = m;
  __syncthreads();
  m = s_red[0];
#pragma unroll
  for (int i = 1; i < 8; ++i) m = fmaxf(m, s_red[i]);
  const float eps = h2f(f2h(1e-5f));
  const float sf = h2f(f2h(__fdiv_rn(fmaxf(m, eps), 127.0f)));
  const RowQuant rq = make_row_quant(sf);
  if (threadIdx.x == 0) scale[blockIdx.x] = sf;
  const __half* hr = h + src_row * C;
  int8_t* qr = q + (size_t)blockIdx.x * C;
  for (int v = threadIdx.x; v < (C >> 3); v += 256) {
    uint4 raw = *reinterpret_cast<const uint4*>(hr + v * 8);
    *reinterpret_cast<uint2*>(qr + v * 8) = quant8_pack(raw, rq);
  }
}

static size_t up256(size_t x) { return (x + 255) & ~size_t(255); }
static int padded_tokens(int T) { return (T + kMoeSegmentAlign - 1) / kMoeSegmentAlign * kMoeSegmentAlign; }

}  // namespace mp

using namespace mp;

// Workspace: plan ints | replicated codes i8 [P, H] | replicated scales f32 [P] | h f16 [P, C] |
// max|h| f32 [P, ceil(C / 128)]; P = chunks * (T rounded up to 256), every part 256-byte aligned.
extern "C" size_t mp_w8a8_gate_up_swiglu_requant_workspace_bytes(int T, int H, int C, int chunks) {
  if (T <= 0 || H <= 0 || C <= 0 || chunks <= 0) return 0;
  const size_t P = (size_t)chunks * padded_tokens(T);
  return up256((1 + P / kMoeTileRows) * sizeof(int)) + up256(P * H) + up256(P * 4) + up256(P * C * 2) +
         up256(P * moe_absmax_slots(C) * 4);
}

extern "C" int mp_w8a8_gate_up_swiglu_requant(const void* x_i8, const void* x_scale_f32, const void* w_i8,
                                              const void* w_scale_f32, int T, int H, int C, int chunks,
                                              void* q_out_i8, void* scale_out_f32, void* workspace,
                                              size_t workspace_bytes, int* error_word, mp_stream_t stream) {
  if (!x_i8 || !x_scale_f32 || !w_i8 || !w_scale_f32 || !q_out_i8 || !scale_out_f32 || T <= 0 || H <= 0 || C <= 0 ||
      chunks <= 0)
    return MP_ERR_INVALID_ARG;
  if (H % 16 != 0 || C % 16 != 0 || chunks > 256) return MP_ERR_UNSUPPORTED;
  const size_t P = (size_t)chunks * padded_tokens(T);
  if (P > (size_t)1 << 30) return MP_ERR_UNSUPPORTED;
  if (!workspace || workspace_bytes < mp_w8a8_gate_up_swiglu_requant_workspace_bytes(T, H, C, chunks))
    return MP_ERR_WORKSPACE;
  if (!aligned(workspace, 256) || !aligned(x_i8, 16) || !aligned(w_i8, 16) || !aligned(q_out_i8, 16))
    return MP_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const int t_pad = padded_tokens(T);
  unsigned char* ws = static_cast<unsigned char*>(workspace);
  int* plan = reinterpret_cast<int*>(ws);
  ws += up256((1 + P / kMoeTileRows) * sizeof(int));
  int8_t* x_rep = reinterpret_cast<int8_t*>(ws);
  ws += up256(P * H);
  float* scale_rep = reinterpret_cast<float*>(ws);
  ws += up256(P * 4);
  __half* h = reinterpret_cast<__half*>(ws);
  ws += up256(P * C * 2);
  float* absmax = reinterpret_cast<float*>(ws);
  int rc = launch_chained(chunk_stage_kernel, dim3((unsigned)P), dim3(256), 0, st, static_cast<const uint4*>(x_i8),
                          static_cast<const float*>(x_scale_f32), T, t_pad, H / 16, chunks,
                          reinterpret_cast<uint4*>(x_rep), scale_rep, plan);
  if (rc != MP_OK) return rc;
  rc = launch_moe_gemm1_swiglu(x_rep, scale_rep, w_i8, static_cast<const float*>(w_scale_f32), (int)P, H, C,
                                   chunks, plan, plan + 1, h, absmax, error_word, st);
  if (rc != MP_OK) return rc;
  return launch_chained(chunk_requant_kernel, dim3((unsigned)(chunks * T)), dim3(256), 0, st, h, absmax,
                        moe_absmax_slots(C), T, t_pad, C, static_cast<int8_t*>(q_out_i8),
                        static_cast<float*>(scale_out_f32));
}
