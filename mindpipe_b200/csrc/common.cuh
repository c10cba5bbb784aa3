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

// ---- programmatic dependent launch for chains of short kernels -------------
// With the process-wide switch on (mp_set_programmatic_launch), launch_chained() lets a kernel be scheduled
// while the previous kernel of the stream is still running; the kernel itself waits for that kernel's results
// with chain_wait() before it reads or writes anything the stream ordered, and chain_release() lets the next
// one be scheduled in turn.  Without the attribute both instructions do nothing.
bool decode_programmatic_launch();   // w4a16_decode_tma.cu

#ifdef __CUDACC__
__device__ __forceinline__ void chain_wait() { asm volatile("griddepcontrol.wait;" ::: "memory"); }
__device__ __forceinline__ void chain_release() { asm volatile("griddepcontrol.launch_dependents;" ::: "memory"); }

template <typename... KArgs, typename... Args>
int launch_chained(void (*kernel)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
  cudaLaunchConfig_t cfg{};
  cfg.gridDim = grid;
  cfg.blockDim = block;
  cfg.dynamicSmemBytes = smem;
  cfg.stream = st;
  cudaLaunchAttribute attrs[1];
  attrs[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
  attrs[0].val.programmaticStreamSerializationAllowed = 1;
  cfg.attrs = attrs;
  cfg.numAttrs = decode_programmatic_launch() ? 1 : 0;
  MP_CUDA_TRY(cudaLaunchKernelEx(&cfg, kernel, static_cast<KArgs>(args)...));
  return MP_OK;
}
#endif

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

// ---- per-row int8 codes of fp16 values: code = rint(f16(x / s)), as torch computes
// x.div_(scale).round_() on an fp16 tensor (fp32 division, rounded to fp16, rounded to an integer).
// For fp16 x and s the fp32 rounding in the middle never changes the result (x / s cannot come within
// 2^-23 relative of an fp16 rounding midpoint without hitting it), so the task is the correctly
// rounded fp16 quotient.  Two routes produce it:
//
//  * packed route (scales >= 2^-14, i.e. every row whose abs-max is above 0.0078): all in f16x2
//    arithmetic, two values per instruction.  With s' = s * 2^-e in [1, 2), x' = x * 2^-e and
//    r = f16(1 / s'):  q = x' * r;  rem = fma(-q, s', x');  q' = fma(rem, r, q).  q' equals the
//    correctly rounded x' / s' for every pair of 11-bit significands with 0.25 <= |x'/s'| <= 128 (checked
//    exhaustively on the CPU; smaller quotients give code 0 on any route).  rint is the addition of
//    1536 = 1.5 * 2^10, after which the code is the low byte of each half.
//  * fp32 route (tiny scales, where 2^-e is not an fp16 number): x * (1/s) in fp32 is within 3 ulps
//    of the correctly rounded quotient and rounds to the same fp16 value unless it lies within 8 fp32
//    ulps of an fp16 rounding midpoint; only then is the IEEE division carried out.
// Row-parallel decode: the kernel leaves its fp32 partial sums in this GPU's own buffer
// ([M][N]) and, once every block has stored, raises this rank's arrival word on every peer
// (flags[q] = rank q's arrival words [world]); the peers then read the buffer over NVLink.
constexpr int kMaxPeerRanks = 16;
struct DecodePush {
  float* partial[2];         // this rank's two buffers (peer-mapped memory), used alternately
  unsigned int* flags[kMaxPeerRanks];
  int* block_counter;        // local device int, zero between calls
  unsigned int* epoch;       // local device word: number of calls completed (this call is *epoch + 1)
  int world, rank;
};

constexpr float kRoundMagic = 12582912.0f;   // 1.5 * 2^23: (v + magic) holds rint(v) in its low mantissa bits

struct RowQuant {
  float s, inv;                 // scale and its fp32 reciprocal (fp32 route)
  __half2 pow2, rcp, neg_sp;    // 2^-e, f16(1 / s'), -s' (packed route)
  __half2 s2;                   // scale, both halves
  bool packed;
};

__device__ __forceinline__ RowQuant make_row_quant(float s) {   // s > 0, an fp16 value held in fp32
  RowQuant rq;
  rq.s = s;
  rq.inv = __frcp_rn(s);
  const int e = static_cast<int>(__float_as_uint(s) >> 23) - 127;
  rq.packed = e >= -14;
  const float p = __uint_as_float(static_cast<uint32_t>(127 - e) << 23);   // 2^-e
  const float sp = s * p;                                                    // exact, in [1, 2)
  rq.pow2 = __float2half2_rn(p);
  rq.rcp = __float2half2_rn(__frcp_rn(sp));
  rq.neg_sp = __float2half2_rn(-sp);
  rq.s2 = __float2half2_rn(s);
  return rq;
}

// Packed route: two values -> f16x2 holding 1536 + code in each half.
__device__ __forceinline__ __half2 quant_pair_packed(__half2 x, const RowQuant& rq) {
  const __half2 xp = __hmul2_rn(x, rq.pow2);
  const __half2 q = __hmul2_rn(xp, rq.rcp);
  const __half2 rem = __hfma2(q, rq.neg_sp, xp);
  const __half2 q2 = __hfma2(rem, rq.rcp, q);
  return __hadd2_rn(q2, __float2half2_rn(1536.0f));
}

__device__ __forceinline__ float quotient_for_f16(float x, float s, float inv_s) {
  float c = x * inv_s;
  const uint32_t low = __float_as_uint(c) & 0x1FFFu;        // the 13 mantissa bits fp16 drops
  if ((low - 0x0FF8u) <= 0x10u) {                           // within 8 ulps of the midpoint 0x1000
    if (fabsf(c) >= 0.25f) c = __fdiv_rn(x, s);
  }
  return c;
}

// fp32 route: two values -> (code + kRoundMagic) each; the code is the low byte of each bit pattern.
__device__ __forceinline__ float2 quant_pair_biased(__half2 h, float s, float inv_s) {
  const float2 x = __half22float2(h);
  const float c0 = quotient_for_f16(x.x, s, inv_s);
  const float c1 = quotient_for_f16(x.y, s, inv_s);
  const float2 r = __half22float2(__floats2half2_rn(c0, c1));
  return make_float2(__fadd_rn(r.x, kRoundMagic), __fadd_rn(r.y, kRoundMagic));
}

__device__ __forceinline__ uint32_t pack_biased_codes(float2 a, float2 b) {
  const uint32_t lo = __byte_perm(__float_as_uint(a.x), __float_as_uint(a.y), 0x0040);
  const uint32_t hi = __byte_perm(__float_as_uint(b.x), __float_as_uint(b.y), 0x0040);
  return __byte_perm(lo, hi, 0x5410);
}

__device__ __forceinline__ uint32_t h2_bits(__half2 h) { return *reinterpret_cast<uint32_t*>(&h); }

// Eight fp16 values (one 128-bit load) -> eight packed int8 codes.
__device__ __forceinline__ uint2 quant8_pack(const uint4& raw, const RowQuant& rq) {
  const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
  if (rq.packed) {
    const uint32_t a = h2_bits(quant_pair_packed(h2[0], rq)), b = h2_bits(quant_pair_packed(h2[1], rq));
    const uint32_t c = h2_bits(quant_pair_packed(h2[2], rq)), d = h2_bits(quant_pair_packed(h2[3], rq));
    return make_uint2(__byte_perm(a, b, 0x6420), __byte_perm(c, d, 0x6420));
  }
  const float2 a = quant_pair_biased(h2[0], rq.s, rq.inv), b = quant_pair_biased(h2[1], rq.s, rq.inv);
  const float2 c = quant_pair_biased(h2[2], rq.s, rq.inv), d = quant_pair_biased(h2[3], rq.s, rq.inv);
  return make_uint2(pack_biased_codes(a, b), pack_biased_codes(c, d));
}

// Same, also producing the fake-quantised values f16(code * s).  Their sign is the input's (s > 0),
// which restores the -0 that round_() keeps for small negative quotients and the biased addition loses.
__device__ __forceinline__ uint2 quant8_pack_fake(const uint4& raw, const RowQuant& rq, uint4& fake) {
  const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
  const uint32_t* xin = reinterpret_cast<const uint32_t*>(&raw);
  uint32_t* fo = reinterpret_cast<uint32_t*>(&fake);
  if (rq.packed) {
    uint32_t w[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) {
      const __half2 b = quant_pair_packed(h2[j], rq);
      w[j] = h2_bits(b);
      const __half2 f = __hmul2_rn(__hsub2_rn(b, __float2half2_rn(1536.0f)), rq.s2);
      fo[j] = (h2_bits(f) & 0x7FFF7FFFu) | (xin[j] & 0x80008000u);
    }
    return make_uint2(__byte_perm(w[0], w[1], 0x6420), __byte_perm(w[2], w[3], 0x6420));
  }
  float2 b[4];
#pragma unroll
  for (int j = 0; j < 4; ++j) {
    b[j] = quant_pair_biased(h2[j], rq.s, rq.inv);
    const __half2 f = __floats2half2_rn(__fmul_rn(__fsub_rn(b[j].x, kRoundMagic), rq.s),
                                        __fmul_rn(__fsub_rn(b[j].y, kRoundMagic), rq.s));
    fo[j] = (h2_bits(f) & 0x7FFF7FFFu) | (xin[j] & 0x80008000u);
  }
  return make_uint2(pack_biased_codes(b[0], b[1]), pack_biased_codes(b[2], b[3]));
}

// max |x| over eight fp16 values, folded into a running half2 maximum.
__device__ __forceinline__ __half2 absmax8(__half2 running, const uint4& raw) {
  const __half2* h2 = reinterpret_cast<const __half2*>(&raw);
#pragma unroll
  for (int j = 0; j < 4; ++j) running = __hmax2(running, __habs2(h2[j]));
  return running;
}
__device__ __forceinline__ float absmax_to_float(__half2 m) {
  const float2 f = __half22float2(m);
  return fmaxf(f.x, f.y);
}

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
