// W4A16 weight-side kernels: asymmetric group quantise + pack, dequantise
// (the bit-exact check of the GEMMs' dequant stage) and the one-time
// re-layout of scales / zero points for the GEMM kernels.
#include "common.cuh"

namespace mp {

// One warp per (row, group); a block of 8 warps covers 8 consecutive groups
// of one row so that it can also emit the packed zero-point word.
// Arithmetic follows pseudo_quantize_tensor(zero_point=True) in
// algorithm/quantization/ptq/awq/source/awq/quantize/quantizer.py:72-97,
// every op rounded to fp16 as torch does on fp16 tensors.
__global__ void __launch_bounds__(256)
w4_quantize_kernel(const __half* __restrict__ w, int N, int K, int group, int groups,
                   uint32_t* __restrict__ packed, __half* __restrict__ scale,
                   uint32_t* __restrict__ zero_words) {
  __shared__ uint32_t s_zero[8];
  const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
  const int n = blockIdx.y;
  const int g = blockIdx.x * 8 + warp;
  if (threadIdx.x < 8) s_zero[threadIdx.x] = 0;
  __syncthreads();
  if (g < groups) {
    const __half* row = w + (size_t)n * K + (size_t)g * group;
    const int chunks = group >> 3;  // 8 columns (16 bytes) per chunk
    float vmax = -INFINITY, vmin = INFINITY;
    for (int c = lane; c < chunks; c += 32) {
      uint4 raw = *reinterpret_cast<const uint4*>(row + c * 8);
      const __half* h = reinterpret_cast<const __half*>(&raw);
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float f = h2f(h[j]);
        vmax = fmaxf(vmax, f);
        vmin = fminf(vmin, f);
      }
    }
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
      vmax = fmaxf(vmax, __shfl_xor_sync(0xffffffffu, vmax, o));
      vmin = fminf(vmin, __shfl_xor_sync(0xffffffffu, vmin, o));
    }
    const __half hmax = f2h(vmax), hmin = f2h(vmin);  // exact: both are fp16 values
    __half span = hsub_t(hmax, hmin);
    const __half eps = f2h(1e-5f);
    if (h2f(span) < h2f(eps)) span = eps;                       // clamp(min=1e-5)
    const __half s = hdiv_t(span, f2h(15.0f));                  // / max_int
    float zf = -rintf(h2f(hdiv_t(hmin, s)));                    // -round(min / scales)
    zf = fminf(fmaxf(zf, 0.0f), 15.0f);                         // clamp_(0, 15)
    for (int c = lane; c < chunks; c += 32) {
      uint4 raw = *reinterpret_cast<const uint4*>(row + c * 8);
      const __half* h = reinterpret_cast<const __half*>(&raw);
      uint32_t word = 0;
#pragma unroll
      for (int j = 0; j < 8; ++j) {
        float q = rintf(h2f(hdiv_t(h[j], s)));                  // round(w / scales), may be +-inf
        q = h2f(f2h(q + zf));                                   // + zeros, rounded to fp16
        q = fminf(fmaxf(q, 0.0f), 15.0f);                       // clamp(0, 15)
        word |= static_cast<uint32_t>(q) << (4 * j);
      }
      packed[(size_t)n * (K >> 3) + (size_t)g * chunks + c] = word;
    }
    if (lane == 0) {
      scale[(size_t)n * groups + g] = s;
      s_zero[warp] = static_cast<uint32_t>(zf);
    }
  }
  __syncthreads();
  if (threadIdx.x == 0) {
    uint32_t zw = 0;
#pragma unroll
    for (int j = 0; j < 8; ++j) zw |= (s_zero[j] & 0xFu) << (4 * j);
    zero_words[(size_t)n * ((groups + 7) >> 3) + blockIdx.x] = zw;
  }
}

__device__ __forceinline__ __half zero_point_of(const uint32_t* zero_words, int n, int groups, int g) {
  if (zero_words == nullptr) return __float2half_rn(8.0f);
  uint32_t zw = zero_words[(size_t)n * ((groups + 7) >> 3) + (g >> 3)];
  return __float2half_rn(static_cast<float>((zw >> (4 * (g & 7))) & 0xFu));
}

// One thread per packed word: 8 codes -> 8 fp16 values (16 bytes), through the
// same dequant8 the GEMM kernels use.
__global__ void __launch_bounds__(256)
w4_dequant_kernel(const uint32_t* __restrict__ packed, const __half* __restrict__ scale,
                  const uint32_t* __restrict__ zero_words, int N, int K, int group, int groups,
                  __half* __restrict__ out) {
  const size_t words_per_row = K >> 3;
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)N * words_per_row) return;
  const int n = static_cast<int>(idx / words_per_row);
  const int c = static_cast<int>(idx % words_per_row);
  const int g = (c * 8) / group;
  const ScaleZero p = make_scale_zero(scale[(size_t)n * groups + g], zero_point_of(zero_words, n, groups, g));
  __half2 v[4];
  dequant8(packed[idx], p, v);
  // v = (k0,k4) (k1,k5) (k2,k6) (k3,k7) -> natural order
  uint32_t a = h2_as_u32(v[0]), b = h2_as_u32(v[1]), cc = h2_as_u32(v[2]), d = h2_as_u32(v[3]);
  uint4 o;
  o.x = prmt(a, b, 0x5410);   // (k0, k1)
  o.y = prmt(cc, d, 0x5410);  // (k2, k3)
  o.z = prmt(a, b, 0x7632);   // (k4, k5)
  o.w = prmt(cc, d, 0x7632);  // (k6, k7)
  *reinterpret_cast<uint4*>(out + idx * 8) = o;
}

// sz[g, n] = (scale[n, g], f16(zero[n, g]))
__global__ void __launch_bounds__(256)
w4_prepare_kernel(const __half* __restrict__ scale, const uint32_t* __restrict__ zero_words,
                  int N, int groups, __half2* __restrict__ sz) {
  const size_t idx = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
  if (idx >= (size_t)N * groups) return;
  const int g = static_cast<int>(idx / N);
  const int n = static_cast<int>(idx % N);
  sz[idx] = __halves2half2(scale[(size_t)n * groups + g], zero_point_of(zero_words, n, groups, g));
}

}  // namespace mp

using namespace mp;

extern "C" int mp_w4a16_quantize(const void* w_f16, int N, int K, int group, void* packed_i32,
                                 void* scale_f16, void* zero_i32, mp_stream_t stream) {
  if (!w_f16 || !packed_i32 || !scale_f16 || !zero_i32 || N <= 0 || K <= 0 || group <= 0) return MP_ERR_INVALID_ARG;
  if (K % 8 != 0 || group % 8 != 0 || K % group != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(w_f16, 16)) return MP_ERR_ALIGNMENT;
  const int groups = K / group;
  dim3 grid((groups + 7) / 8, N);
  w4_quantize_kernel<<<grid, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(w_f16), N, K, group, groups, static_cast<uint32_t*>(packed_i32),
      static_cast<__half*>(scale_f16), static_cast<uint32_t*>(zero_i32));
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" int mp_w4a16_dequant(const void* packed_i32, const void* scale_f16, const void* zero_i32,
                                int N, int K, int group, void* w_out_f16, mp_stream_t stream) {
  if (!packed_i32 || !scale_f16 || !w_out_f16 || N <= 0 || K <= 0 || group <= 0) return MP_ERR_INVALID_ARG;
  if (K % 8 != 0 || group % 8 != 0 || K % group != 0) return MP_ERR_UNSUPPORTED;
  if (!aligned(w_out_f16, 16)) return MP_ERR_ALIGNMENT;
  const size_t words = (size_t)N * (K / 8);
  const unsigned blocks = static_cast<unsigned>((words + 255) / 256);
  w4_dequant_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const uint32_t*>(packed_i32), static_cast<const __half*>(scale_f16),
      static_cast<const uint32_t*>(zero_i32), N, K, group, K / group, static_cast<__half*>(w_out_f16));
  MP_LAUNCH_CHECK();
  return MP_OK;
}

extern "C" int mp_w4a16_prepare(const void* scale_f16, const void* zero_i32, int N, int K, int group,
                                void* sz_f16x2, mp_stream_t stream) {
  if (!scale_f16 || !sz_f16x2 || N <= 0 || K <= 0 || group <= 0) return MP_ERR_INVALID_ARG;
  if (K % group != 0) return MP_ERR_UNSUPPORTED;
  const int groups = K / group;
  const size_t total = (size_t)N * groups;
  const unsigned blocks = static_cast<unsigned>((total + 255) / 256);
  w4_prepare_kernel<<<blocks, 256, 0, static_cast<cudaStream_t>(stream)>>>(
      static_cast<const __half*>(scale_f16), static_cast<const uint32_t*>(zero_i32), N, groups,
      static_cast<__half2*>(sz_f16x2));
  MP_LAUNCH_CHECK();
  return MP_OK;
}
