// Shared helpers for the sm_100a kernels: status codes, launch checks and the
// fp16 arithmetic that reproduces torch's CPU half semantics bit for bit.
#pragma once

#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/mindpipe_b200.h"

namespace mp {

extern thread_local int g_last_cuda_error;

inline int cuda_fail(cudaError_t e) {
  g_last_cuda_error = static_cast<int>(e);
  return MP_ERR_CUDA;
}

#define MP_CUDA_TRY(expr)                                 \
  do {                                                    \
    cudaError_t _e = (expr);                              \
    if (_e != cudaSuccess) return ::mp::cuda_fail(_e);    \
  } while (0)

#define MP_LAUNCH_CHECK() MP_CUDA_TRY(cudaGetLastError())

inline bool aligned(const void* p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }

constexpr int kSmCount = 148;  // B200

// ---- fp16 arithmetic as torch evaluates it on the CPU ----------------------
// torch computes each elementwise half op as half(op(float(a), float(b))).
// Every helper below widens, applies the IEEE fp32 op with round-to-nearest,
// and rounds once to half, so results match the reference bit for bit
// (including the double rounding of inexact fp32 results).
__device__ __forceinline__ float h2f(__half h) { return __half2float(h); }
__device__ __forceinline__ __half f2h(float f) { return __float2half_rn(f); }
__device__ __forceinline__ __half hdiv_t(__half a, __half b) { return f2h(__fdiv_rn(h2f(a), h2f(b))); }
__device__ __forceinline__ __half hsub_t(__half a, __half b) { return f2h(__fsub_rn(h2f(a), h2f(b))); }
__device__ __forceinline__ __half hadd_t(__half a, __half b) { return f2h(__fadd_rn(h2f(a), h2f(b))); }
__device__ __forceinline__ __half hmul_t(__half a, __half b) { return f2h(__fmul_rn(h2f(a), h2f(b))); }

// ---- int4 -> fp16 dequantisation ------------------------------------------
// One packed word holds the codes of columns 8c..8c+7, low nibble first.
// dequant8 returns them as four half2 in the order
//   v[0]=(k0,k4) v[1]=(k1,k5) v[2]=(k2,k6) v[3]=(k3,k7)
// each element being exactly f16((u - z) * s): the code is planted in the
// mantissa of 1024.0 (or of 1024 + 16u for the odd nibbles), the zero point
// is removed exactly, and a single fp16 multiply rounds once.
struct ScaleZero {
  __half2 s2;       // (s, s)
  __half2 z_lo;     // (1024 + z) twice
  __half2 z_hi;     // -(64 + z) twice
};

__device__ __forceinline__ ScaleZero make_scale_zero(__half s, __half z) {
  ScaleZero r;
  r.s2 = __half2half2(s);
  // z is an integer in [0,15], so both sums are exact in fp16.
  r.z_lo = __half2half2(__hadd(__float2half_rn(1024.0f), z));
  r.z_hi = __half2half2(__hneg(__hadd(__float2half_rn(64.0f), z)));
  return r;
}

__device__ __forceinline__ uint32_t lop3_and_or(uint32_t a, uint32_t mask, uint32_t orv) {
  uint32_t r;
  asm("lop3.b32 %0, %1, %2, %3, 0xea;" : "=r"(r) : "r"(a), "r"(mask), "r"(orv));  // (a & mask) | orv
  return r;
}

__device__ __forceinline__ void dequant8(uint32_t q, const ScaleZero& p, __half2 (&v)[4]) {
  const uint32_t kMagic = 0x64006400u;                 // half2(1024, 1024)
  const __half2 k16th = __float2half2_rn(0.0625f);
  uint32_t lo0 = lop3_and_or(q, 0x000f000fu, kMagic);  // 1024 + (u0, u4)
  uint32_t hi0 = lop3_and_or(q, 0x00f000f0u, kMagic);  // 1024 + 16 * (u1, u5)
  q >>= 8;
  uint32_t lo1 = lop3_and_or(q, 0x000f000fu, kMagic);  // (u2, u6)
  uint32_t hi1 = lop3_and_or(q, 0x00f000f0u, kMagic);  // (u3, u7)
  __half2 d0 = __hsub2(*reinterpret_cast<__half2*>(&lo0), p.z_lo);
  __half2 d1 = __hfma2(*reinterpret_cast<__half2*>(&hi0), k16th, p.z_hi);
  __half2 d2 = __hsub2(*reinterpret_cast<__half2*>(&lo1), p.z_lo);
  __half2 d3 = __hfma2(*reinterpret_cast<__half2*>(&hi1), k16th, p.z_hi);
  v[0] = __hmul2(d0, p.s2);
  v[1] = __hmul2(d1, p.s2);
  v[2] = __hmul2(d2, p.s2);
  v[3] = __hmul2(d3, p.s2);
}

__device__ __forceinline__ uint32_t h2_as_u32(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel) {
  uint32_t r;
  asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
  return r;
}

// Streaming 128-bit load that does not pollute L1 (weights are read once).
__device__ __forceinline__ uint4 ldg_stream_v4(const void* p) {
  uint4 r;
  asm volatile("ld.global.nc.L1::no_allocate.v4.u32 {%0,%1,%2,%3}, [%4];"
               : "=r"(r.x), "=r"(r.y), "=r"(r.z), "=r"(r.w)
               : "l"(p));
  return r;
}

}  // namespace mp
