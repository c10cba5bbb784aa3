// Per-row (token / output channel) symmetric int8 quantisation.
//
// Arithmetic of quantize_activation_per_token_absmax and
// quantize_weight_per_channel_absmax
// (algorithm/quantization/ptq/smoothquant/source/smoothquant/fake_quant.py:10-31)
// with the integer codes kept, which is what npu_dynamic_quant returns at
// acceleration/runtime_patches/vllm_ascend.patch:3950:
//   s    = f16( max(absmax, f16(1e-5)) / 127 )
//   code = rint( f16( x / s ) )         (division in fp32, rounded to fp16 first)
//   fake = f16( code * s )
// The row is read with 128-bit loads, reduced with warp shuffles and kept in
// registers for the rounding step (rows up to 16384 columns), so it is read once.
#include "common.cuh"

namespace mp {

// Quantise eight values held in one 128-bit register group and store the codes and / or the
// fake-quantised values f16(code * s).
__device__ __forceinline__ void emit_codes(const uint4& raw, const RowQuant& rq, int8_t* q8, __half* fake8) {
  if (fake8) {
    uint4 fk;
    const uint2 codes = quant8_pack_fake(raw, rq, fk);
    if (q8) *reinterpret_cast<uint2*>(q8) = codes;
    *reinterpret_cast<uint4*>(fake8) = fk;
  } else if (q8) {
    *reinterpret_cast<uint2*>(q8) = quant8_pack(raw, rq);
  }
}

// One warp per row (rows of up to 32 * 8 * NV columns): the row is read once with NV independent
// 128-bit loads per lane, reduced with shuffles only, and quantised from registers -- no block-level
// synchronisation at all.
// CODES / FAKE select the outputs at compile time and the rare tiny-scale rows take a rolled loop that
// re-reads the row, so the unrolled body holds one route only (the kernel stays small enough for the
// instruction cache).
template <int NV, bool CODES, bool FAKE>
__global__ void __launch_bounds__(128)
act_quant_warp_kernel(const __half* __restrict__ x, int M, int K, int8_t* __restrict__ q,
                      float* __restrict__ scale, __half* __restrict__ fake) {
  chain_wait();              // programmatic dependent launch: the producer of x has finished
  chain_release();
  const int row = blockIdx.x * 4 + (threadIdx.x >> 5);
  if (row >= M) return;
  const int lane = threadIdx.x & 31;
  const __half* xr = x + (size_t)row * K;
  const int chunks = K >> 3;
  uint4 held[NV];
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int c = lane + v * 32;
    held[v] = c < chunks ? *reinterpret_cast<const uint4*>(xr + c * 8) : make_uint4(0, 0, 0, 0);
  }
  __half2 m2 = __float2half2_rn(0.0f);
#pragma unroll
  for (int v = 0; v < NV; ++v) m2 = absmax8(m2, held[v]);
  float amax = absmax_to_float(m2);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  const float eps = h2f(f2h(1e-5f));                                   // clamp_(min=1e-5) on an fp16 tensor
  const float sf = h2f(f2h(__fdiv_rn(fmaxf(amax, eps), 127.0f)));      // div_(q_max), rounded to fp16
  RowQuant rq = make_row_quant(sf);
  if (lane == 0 && scale) scale[row] = sf;
  int8_t* qr = CODES ? q + (size_t)row * K : nullptr;
  __half* fr = FAKE ? fake + (size_t)row * K : nullptr;
  if (!rq.packed) {                                   // scale below 2^-14: fp32 route, rolled
#pragma unroll 1
    for (int c = lane; c < chunks; c += 32)
      emit_codes(*reinterpret_cast<const uint4*>(xr + c * 8), rq, CODES ? qr + c * 8 : nullptr,
                 FAKE ? fr + c * 8 : nullptr);
    return;
  }
  rq.packed = true;                                   // lets the compiler drop the other route below
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int c = lane + v * 32;
    if (c >= chunks) continue;
    emit_codes(held[v], rq, CODES ? qr + c * 8 : nullptr, FAKE ? fr + c * 8 : nullptr);
  }
}

template <int NV>
static int launch_act_quant_warp(const __half* x, int M, int K, int8_t* q, float* sc, __half* fk, cudaStream_t st) {
  const unsigned blocks = static_cast<unsigned>((M + 3) / 4);
  if (q && fk) {
    return launch_chained(act_quant_warp_kernel<NV, true, true>, dim3(blocks), dim3(128), 0, st, x, M, K, q, sc, fk);
  } else if (q) {
    return launch_chained(act_quant_warp_kernel<NV, true, false>, dim3(blocks), dim3(128), 0, st, x, M, K, q, sc, fk);
  } else {
    return launch_chained(act_quant_warp_kernel<NV, false, true>, dim3(blocks), dim3(128), 0, st, x, M, K, q, sc, fk);
  }
}

// NV = 128-bit vectors per thread.  NV > 0: the row (K <= THREADS * 8 * NV) is held in
// registers between the abs-max and the rounding step, so global memory is read once;
// NV == 0: any K, second pass re-reads the row (an L1/L2 hit).
template <int THREADS, int NV>
__global__ void __launch_bounds__(THREADS)
act_quant_kernel(const __half* __restrict__ x, int M, int K, int8_t* __restrict__ q,
                 float* __restrict__ scale, __half* __restrict__ fake) {
  chain_wait();
  chain_release();
  __shared__ float s_red[THREADS / 32];
  __shared__ float s_scale;
  const int row = blockIdx.x;
  const __half* xr = x + (size_t)row * K;
  const int chunks = K >> 3;
  constexpr int NREG = NV > 0 ? NV : 1;
  uint4 held[NREG];
  __half2 m2 = __float2half2_rn(0.0f);
  auto absmax_of = [&](const uint4& raw) { m2 = absmax8(m2, raw); };
  if (NV > 0) {
#pragma unroll
    for (int v = 0; v < NREG; ++v) {
      const int c = threadIdx.x + v * THREADS;
      held[v] = c < chunks ? *reinterpret_cast<const uint4*>(xr + c * 8) : make_uint4(0, 0, 0, 0);
    }
#pragma unroll
    for (int v = 0; v < NREG; ++v) absmax_of(held[v]);
  } else {
    for (int c = threadIdx.x; c < chunks; c += THREADS) absmax_of(*reinterpret_cast<const uint4*>(xr + c * 8));
  }
  float amax = absmax_to_float(m2);
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, o));
  if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = amax;
  __syncthreads();
  if (threadIdx.x < 32) {
    float v = threadIdx.x < THREADS / 32 ? s_red[threadIdx.x] : 0.0f;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    if (threadIdx.x == 0) {
      const float eps = h2f(f2h(1e-5f));                      // clamp_(min=1e-5) on an fp16 tensor
      const __half s = f2h(__fdiv_rn(fmaxf(v, eps), 127.0f)); // div_(q_max), rounded to fp16
      s_scale = h2f(s);
      if (scale) scale[row] = s_scale;
    }
  }
  __syncthreads();
  const RowQuant rq = make_row_quant(s_scale);
  auto emit = [&](int c, const uint4& raw) {
    emit_codes(raw, rq, q ? q + (size_t)row * K + c * 8 : nullptr,
               fake ? fake + (size_t)row * K + c * 8 : nullptr);
  };
  if (NV > 0) {
#pragma unroll
    for (int v = 0; v < NREG; ++v) {
      const int c = threadIdx.x + v * THREADS;
      if (c < chunks) emit(c, held[v]);
    }
  } else {
    for (int c = threadIdx.x; c < chunks; c += THREADS) emit(c, *reinterpret_cast<const uint4*>(xr + c * 8));
  }
}

// OmniQuant-style dynamic asymmetric quantisation of each row to unsigned 8-bit codes:
// UniformAffineQuantizer.per_token_dynamic_calibration + fake_quant
// (algorithm/quantization/ptq/omniquant/source/omniquant/quantizer.py:124-150, 89-111;
// symmetric=False, no group, no learned clipping), every op rounded to fp16 as torch does:
//   s  = clamp(f16(f16(max - min) / 255), 1e-5, 1e4)
//   zp = rint(clamp(f16(-min / s), -1e4, 1e4))
//   u  = clamp(f16(rint(f16(x / s)) + zp), 0, 255);   fake = f16(f16(u - zp) * s)
// Also emits the row sum of the codes, which the integer GEMM's zero-point correction needs.
template <int THREADS>
__global__ void __launch_bounds__(THREADS)
affine_quant_kernel(const __half* __restrict__ x, int K, uint8_t* __restrict__ q, float* __restrict__ scale,
                    float* __restrict__ zero, int* __restrict__ rowsum, __half* __restrict__ fake) {
  __shared__ float s_max[THREADS / 32], s_min[THREADS / 32];
  __shared__ int s_sum[THREADS / 32];
  __shared__ float s_scale, s_zp;
  const int row = blockIdx.x;
  const __half* xr = x + (size_t)row * K;
  const int chunks = K >> 3;
  float vmax = -INFINITY, vmin = INFINITY;
  for (int c = threadIdx.x; c < chunks; c += THREADS) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xr + c * 8);
    const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      const float f = h2f(h[j]);
      vmax = fmaxf(vmax, f);
      vmin = fminf(vmin, f);
    }
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) {
    vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
    vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, o));
  }
  if ((threadIdx.x & 31) == 0) { s_max[threadIdx.x >> 5] = vmax; s_min[threadIdx.x >> 5] = vmin; }
  __syncthreads();
  if (threadIdx.x == 0) {
    for (int i = 1; i < THREADS / 32; ++i) { vmax = fmaxf(vmax, s_max[i]); vmin = fminf(vmin, s_min[i]); }
    const __half hmax = f2h(vmax), hmin = f2h(vmin);
    __half s = hdiv_t(hsub_t(hmax, hmin), f2h(255.0f));
    const float lo = h2f(f2h(1e-5f)), hi = h2f(f2h(1e4f));
    s = f2h(fminf(fmaxf(h2f(s), lo), hi));
    float zp = h2f(hdiv_t(__hneg(hmin), s));
    zp = rintf(fminf(fmaxf(zp, -hi), hi));
    s_scale = h2f(s);
    s_zp = zp;
    scale[row] = s_scale;
    zero[row] = zp;
  }
  __syncthreads();
  const float sf = s_scale, zp = s_zp;
  int local_sum = 0;
  for (int c = threadIdx.x; c < chunks; c += THREADS) {
    const uint4 raw = *reinterpret_cast<const uint4*>(xr + c * 8);
    const __half* h = reinterpret_cast<const __half*>(&raw);
    uint32_t w0 = 0, w1 = 0;
    __align__(16) __half out[8];
#pragma unroll
    for (int j = 0; j < 8; ++j) {
      float u = rintf(h2f(f2h(__fdiv_rn(h2f(h[j]), sf))));
      u = h2f(f2h(u + zp));
      u = fminf(fmaxf(u, 0.0f), 255.0f);
      const uint32_t code = static_cast<uint32_t>(u);
      local_sum += static_cast<int>(code);
      if (j < 4) w0 |= code << (8 * j); else w1 |= code << (8 * (j - 4));
      out[j] = hmul_t(f2h(u - zp), f2h(sf));
    }
    if (q) *reinterpret_cast<uint2*>(q + (size_t)row * K + c * 8) = make_uint2(w0, w1);
    if (fake) *reinterpret_cast<uint4*>(fake + (size_t)row * K + c * 8) = *reinterpret_cast<uint4*>(out);
  }
#pragma unroll
  for (int o = 16; o > 0; o >>= 1) local_sum += __shfl_xor_sync(0xffffffffu, local_sum, o);
  if ((threadIdx.x & 31) == 0) s_sum[threadIdx.x >> 5] = local_sum;
  __syncthreads();
  if (threadIdx.x == 0 && rowsum) {
    int tot = 0;
    for (int i = 0; i < THREADS / 32; ++i) tot += s_sum[i];
    rowsum[row] = tot;
  }
}

// Residual add + RMSNorm + per-token int8 quant in one pass over the row: the
// torch_npu.npu_add_rms_norm_dynamic_quant call that feeds the (codes, scale) tuple to
// the W8A8 linear (acceleration/runtime_patches/vllm_ascend.patch:754-770).
//   r   = f16(x + residual)                      (written back as the new residual)
//   y   = f16( f16(r * rsqrt(mean(r^2) + eps)) * gamma )   (RMSNorm as HF Llama computes it)
//   q,s = per-token absmax int8 of y             (same arithmetic as act_quant_kernel)
template <int THREADS, int NV>
__global__ void __launch_bounds__(THREADS)
add_rmsnorm_quant_kernel(const __half* __restrict__ x, __half* __restrict__ residual,
                         const __half* __restrict__ gamma, float eps, int H, int8_t* __restrict__ q,
                         float* __restrict__ scale) {
  __shared__ float s_red[THREADS / 32];
  __shared__ float s_bcast;
  const int row = blockIdx.x;
  const int chunks = H >> 3;
  const __half* xr = x + (size_t)row * H;
  __half* rr = residual + (size_t)row * H;
  auto block_reduce = [&](float v, bool is_max) -> float {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      const float other = __shfl_xor_sync(0xffffffffu, v, o);
      v = is_max ? fmaxf(v, other) : v + other;
    }
    __syncthreads();                               // s_red may still be read from the previous reduction
    if ((threadIdx.x & 31) == 0) s_red[threadIdx.x >> 5] = v;
    __syncthreads();
    if (threadIdx.x < 32) {
      float w = threadIdx.x < THREADS / 32 ? s_red[threadIdx.x] : 0.0f;
#pragma unroll
      for (int o = 16; o > 0; o >>= 1) {
        const float other = __shfl_xor_sync(0xffffffffu, w, o);
        w = is_max ? fmaxf(w, other) : w + other;
      }
      if (threadIdx.x == 0) s_bcast = w;
    }
    __syncthreads();
    return s_bcast;
  };
  uint4 held[NV];
  float sumsq = 0.0f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int c = threadIdx.x + v * THREADS;
    held[v] = make_uint4(0, 0, 0, 0);
    if (c < chunks) {
      const uint4 a = *reinterpret_cast<const uint4*>(xr + c * 8);
      const uint4 b = *reinterpret_cast<const uint4*>(rr + c * 8);
      const __half* ha = reinterpret_cast<const __half*>(&a);
      const __half* hb = reinterpret_cast<const __half*>(&b);
      __align__(16) __half hs[8];
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        hs[j] = hadd_t(ha[j], hb[j]);
        const float f = h2f(hs[j]);
        sumsq += f * f;
      }
      held[v] = *reinterpret_cast<uint4*>(hs);
      *reinterpret_cast<uint4*>(rr + c * 8) = held[v];           // new residual
    }
  }
  const float inv = rsqrtf(block_reduce(sumsq, false) / static_cast<float>(H) + eps);
  float amax = 0.0f;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int c = threadIdx.x + v * THREADS;
    if (c < chunks) {
      const uint4 gw = *reinterpret_cast<const uint4*>(gamma + c * 8);
      const __half* hg = reinterpret_cast<const __half*>(&gw);
      __half* hs = reinterpret_cast<__half*>(&held[v]);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        hs[j] = hmul_t(f2h(h2f(hs[j]) * inv), hg[j]);
        amax = fmaxf(amax, fabsf(h2f(hs[j])));
      }
    }
  }
  const float eps_q = h2f(f2h(1e-5f));
  const float sf = h2f(f2h(__fdiv_rn(fmaxf(block_reduce(amax, true), eps_q), 127.0f)));
  const RowQuant rq = make_row_quant(sf);
  if (threadIdx.x == 0) scale[row] = sf;
#pragma unroll
  for (int v = 0; v < NV; ++v) {
    const int c = threadIdx.x + v * THREADS;
    if (c < chunks) {
      *reinterpret_cast<uint2*>(q + (size_t)row * H + c * 8) = quant8_pack(held[v], rq);
    }
  }
}

}  // namespace mp

using namespace mp;

extern "C" int mp_add_rmsnorm_quant(const void* x_f16, void* residual_f16, const void* gamma_f16, float eps, int M,
                                    int H, void* q_i8, void* scale_f32, mp_stream_t stream) {
  if (!x_f16 || !residual_f16 || !gamma_f16 || !q_i8 || !scale_f32 || M <= 0 || H <= 0) return MP_ERR_INVALID_ARG;
  if (H % 8 != 0 || H > 16384) return MP_ERR_UNSUPPORTED;
  if (!aligned(x_f16, 16) || !aligned(residual_f16, 16) || !aligned(gamma_f16, 16) || !aligned(q_i8, 8)) return MP_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __half* x = static_cast<const __half*>(x_f16);
  __half* r = static_cast<__half*>(residual_f16);
  const __half* g = static_cast<const __half*>(gamma_f16);
  int8_t* q = static_cast<int8_t*>(q_i8);
  float* sc = static_cast<float*>(scale_f32);
  if (H <= 2048) {
    add_rmsnorm_quant_kernel<256, 1><<<M, 256, 0, st>>>(x, r, g, eps, H, q, sc);
  } else if (H <= 4096) {
    add_rmsnorm_quant_kernel<256, 2><<<M, 256, 0, st>>>(x, r, g, eps, H, q, sc);
  } else if (H <= 8192) {
    add_rmsnorm_quant_kernel<512, 2><<<M, 512, 0, st>>>(x, r, g, eps, H, q, sc);
  } else {
    add_rmsnorm_quant_kernel<512, 4><<<M, 512, 0, st>>>(x, r, g, eps, H, q, sc);
  }
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" int mp_act_quant_per_token(const void* x_f16, int M, int K, void* q_i8, void* scale_f32,
                                      void* fake_f16, mp_stream_t stream) {
  if (!x_f16 || M <= 0 || K <= 0 || (!q_i8 && !fake_f16)) return MP_ERR_INVALID_ARG;
  if (K % 8 != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(x_f16, 16) || (q_i8 && !aligned(q_i8, 8)) || (fake_f16 && !aligned(fake_f16, 16))) return MP_ERR_ALIGNMENT;
  cudaStream_t st = static_cast<cudaStream_t>(stream);
  const __half* x = static_cast<const __half*>(x_f16);
  int8_t* q = static_cast<int8_t*>(q_i8);
  float* sc = static_cast<float*>(scale_f32);
  __half* fk = static_cast<__half*>(fake_f16);
  if (K <= 1024) {
    return launch_act_quant_warp<4>(x, M, K, q, sc, fk, st);
  } else if (K <= 2048) {
    return launch_act_quant_warp<8>(x, M, K, q, sc, fk, st);
  } else if (K <= 4096) {
    return launch_act_quant_warp<16>(x, M, K, q, sc, fk, st);
  } else if (K <= 8192) {
    return launch_chained(act_quant_kernel<512, 2>, dim3(M), dim3(512), 0, st, x, M, K, q, sc, fk);
  } else if (K <= 16384) {
    return launch_chained(act_quant_kernel<512, 4>, dim3(M), dim3(512), 0, st, x, M, K, q, sc, fk);
  } else {
    return launch_chained(act_quant_kernel<512, 0>, dim3(M), dim3(512), 0, st, x, M, K, q, sc, fk);
  }
}

extern "C" int mp_affine_quant_per_row(const void* x_f16, int M, int K, void* q_u8, void* scale_f32, void* zero_f32,
                                       void* rowsum_i32, void* fake_f16, mp_stream_t stream) {
  if (!x_f16 || !scale_f32 || !zero_f32 || M <= 0 || K <= 0 || (!q_u8 && !fake_f16)) return MP_ERR_INVALID_ARG;
  if (K % 8 != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(x_f16, 16) || (q_u8 && !aligned(q_u8, 8)) || (fake_f16 && !aligned(fake_f16, 16))) return MP_ERR_ALIGNMENT;
  affine_quant_kernel<256><<<M, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(x_f16), K, static_cast<uint8_t*>(q_u8), static_cast<float*>(scale_f32),
      static_cast<float*>(zero_f32), static_cast<int*>(rowsum_i32), static_cast<__half*>(fake_f16));
  MP_LAUNCH_CHECK();
  return MP_OK;
}
