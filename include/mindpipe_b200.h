/*
 * mindpipe_b200 -- C ABI of the B200 (sm_100a) quantized-linear kernels.
 *
 * Every entry point takes plain device pointers, sizes and a CUDA stream, is
 * asynchronous on that stream, never synchronises, never allocates (scratch
 * comes from the caller, sized by the matching *_workspace_bytes query) and
 * returns 0 or a negative mp_status.  Pointers are borrowed for the call.
 * All matrices are dense row-major; "f16" is IEEE binary16.
 *
 * Each declaration names the reference interface it stands in for, by path
 * inside the MindPipe repository.
 */
#ifndef MINDPIPE_B200_H_
#define MINDPIPE_B200_H_

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

typedef void* mp_stream_t; /* a cudaStream_t */

enum mp_status {
  MP_OK = 0,
  MP_ERR_INVALID_ARG = -1,   /* null pointer, non-positive size */
  MP_ERR_UNSUPPORTED = -2,   /* shape outside what the kernel handles */
  MP_ERR_ALIGNMENT = -3,     /* pointer or row pitch not aligned as required */
  MP_ERR_WORKSPACE = -4,     /* workspace missing or too small */
  MP_ERR_CUDA = -5,          /* a CUDA runtime/driver call failed (see mp_last_cuda_error) */
  MP_ERR_DEVICE = -6         /* a device-side bounded wait gave up (see mp_device_error_word) */
};

int mp_abi_version(void);
const char* mp_status_string(int status);
/* Last cudaError_t seen by this library on the calling thread (0 = none). */
int mp_last_cuda_error(void);

/* ------------------------------------------------------------------ W4A16 */

/*
 * Quantise fp16 weights w[N,K] to asymmetric int4 per group of `group`
 * columns and pack them: the arithmetic of
 *   pseudo_quantize_tensor(w, n_bit=4, zero_point=True, q_group_size=group)
 *   (algorithm/quantization/ptq/awq/source/awq/quantize/quantizer.py:63-105)
 * with the nibble order of pack_int4_for_vllm
 *   (algorithm/quantization/exporters/vllm.py:89-111): nibble j of word c is
 * column 8c+j.  group must divide K (pass group=K for one group per row,
 * the reference's fallback at quantizer.py:67-68); K % 8 == 0.
 *   packed  int32 [N, K/8]        unsigned codes u in [0,15]
 *   scale   f16   [N, K/group]
 *   zero    int32 [N, ceil(K/group/8)]  zero points, same nibble order
 */
int mp_w4a16_quantize(const void* w_f16, int N, int K, int group,
                      void* packed_i32, void* scale_f16, void* zero_i32, mp_stream_t stream);

/*
 * Dequantise to fp16 w_out[N,K] = f16((u - z) * s): the last step of
 * pseudo_quantize_tensor (quantizer.py:95-97), and _dequantize_weight
 * (scripts/repro/evaluate_real_quant_export_dequant.py:46-64) when
 * zero_i32 == NULL (symmetric export format, zero point 8).
 */
int mp_w4a16_dequant(const void* packed_i32, const void* scale_f16, const void* zero_i32,
                     int N, int K, int group, void* w_out_f16, mp_stream_t stream);

/*
 * One-time re-layout of the per-group parameters for the GEMM kernels (the
 * role process_weights_after_loading plays at
 * acceleration/runtime_patches/vllm_ascend.patch:4022-4033): sz[K/group, N]
 * of f16 pairs (scale, zero point as f16), group-major so that a tile of
 * output rows reads it contiguously.  zero_i32 == NULL gives zero point 8.
 */
int mp_w4a16_prepare(const void* scale_f16, const void* zero_i32, int N, int K, int group,
                     void* sz_f16x2, mp_stream_t stream);

/*
 * y[M,N] = x[M,K] @ dequant(W)[N,K]^T (+ bias[N]); fp16 in/out, fp32
 * accumulate.  Stands in for the W4A16 forward of the reference,
 * F.linear(x, pseudo_quantize_tensor(W)) (quantizer.py:109-130), and for the
 * forward VllmPackedInt4Linear leaves unimplemented
 * (algorithm/quantization/exporters/vllm.py:85-86).
 * Decode variant: M <= 64, streams the packed weights once, split over K.
 * Requires K % 128 == 0, group % 32 == 0, N % 8 == 0.  The workspace must be
 * zero-filled once when it is allocated; every call leaves it ready for the
 * next one.  Calls that share a workspace must not overlap on the device.
 */
size_t mp_w4a16_decode_workspace_bytes(int M, int N, int K);
size_t mp_w4a16_decode_workspace_bytes_ex(int M, int N, int K, int k_split);
int mp_w4a16_linear_decode(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                           const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                           void* workspace, size_t workspace_bytes, mp_stream_t stream);
/* Same, with the K split and rows per block chosen by the caller (0 = automatic). */
int mp_w4a16_linear_decode_ex(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                              const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                              void* workspace, size_t workspace_bytes, int k_split,
                              mp_stream_t stream);

/* ------------------------------------------------------------------- W8A8 */

/*
 * Per-token (row) symmetric int8 quantisation:
 *   s = f16(max(absmax, f16(1e-5)) / 127), q = rint(f16(x / s)).
 * The arithmetic of quantize_activation_per_token_absmax
 * (algorithm/quantization/ptq/smoothquant/source/smoothquant/fake_quant.py:22-31)
 * with the integer codes kept, i.e. the torch_npu.npu_dynamic_quant call of
 * AscendW8A8DynamicLinearMethod.apply
 * (acceleration/runtime_patches/vllm_ascend.patch:3950).  Run on weight rows
 * it is quantize_weight_per_channel_absmax (fake_quant.py:10-19).
 *   q_i8 [M,K], scale_f32 [M] (the fp16 scale widened to fp32).  K % 8 == 0.
 * fake_f16 (optional, may be NULL) receives f16(q * s), the fake-quantised
 * tensor the reference module passes on (fake_quant.py:77-88); q_i8 and
 * scale_f32 may be NULL when only fake_f16 is wanted.
 */
int mp_act_quant_per_token(const void* x_f16, int M, int K, void* q_i8, void* scale_f32,
                           void* fake_f16, mp_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MINDPIPE_B200_H_ */
