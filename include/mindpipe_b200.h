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
/*
 * Same, with the K split chosen by the caller.  k_split == 0 is automatic: for
 * M <= 16 a thread-block-cluster kernel that reduces the K split through
 * distributed shared memory and touches no workspace; otherwise (M > 16, or
 * an explicit k_split >= 1) the workspace kernel.
 */
int mp_w4a16_linear_decode_ex(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                              const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                              void* workspace, size_t workspace_bytes, int k_split,
                              mp_stream_t stream);

/*
 * Row-parallel decode linear (the input features K sharded over `world` GPUs, as
 * a tensor-parallel runtime shards down_proj / o_proj; the reference computes
 * the unsharded nn.Linear, quantizer.py:109-130): y = sum over ranks of
 * x[:, K_r] @ dequant(W[:, K_r])^T, M <= 16.
 *   _push    runs the decode kernel on this rank's shard, leaves its fp32
 *            partial sums in one of this rank's two buffers ([M][N] fp32 each,
 *            peer-mapped memory; the call number's parity picks it, because a
 *            peer may still read call n while this rank computes call n+1) and,
 *            once every block has stored, advances the call number in
 *            epoch_counter (device word, zero at start) and raises it as this
 *            rank's arrival word on every peer.  block_counter is a device int
 *            that is zero between calls.
 *   _finish  waits (bounded, 2 s -> error word 5) until all arrival words of
 *            this rank have reached the call number, reads every rank's buffer
 *            over NVLink, adds them in rank order (+bias) and writes fp16:
 *            every rank gets the same bits.
 * No argument changes from call to call, so the pair can sit in a captured CUDA
 * graph (replayed the same number of times on every rank).
 */
int mp_w4a16_rowparallel_push(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                              void* partial0_f32, void* partial1_f32, void* const* peer_flags_u32,
                              int* block_counter, void* epoch_counter_u32, int world, int rank, int M,
                              int N, int K_local, int group, mp_stream_t stream);
int mp_w4a16_rowparallel_finish(void* const* peer_partial0_f32, void* const* peer_partial1_f32,
                                const void* flags_u32, int world, const void* epoch_counter_u32, int M,
                                int N, const void* bias_f16, void* y_f16, int* error_word,
                                mp_stream_t stream);

/*
 * Host-buffer form of the decode linear for M <= 16, for a host that keeps its
 * activations in (preferably pinned) host memory, as the reference's CPU
 * forward does (quantizer.py:109-130 runs nn.Linear on host tensors): copies
 * x_host into x_stage, runs the linear into y_stage and copies the result to
 * y_host, all enqueued on `stream` without blocking; y_host is valid once the
 * stream has been synchronised.  x_stage [M,K] and y_stage [M,N] are device
 * buffers of the caller (nothing is allocated here).
 * y_host_f16 may be NULL: the result then stays in y_stage and no copy is
 * issued.  With y_stage = the device alias of a pinned host buffer
 * (mp_host_buffer_device_alias) the kernel's own stores carry the result to
 * host memory: one call less on the host per linear and no copy node between
 * the kernel and the host's read.
 */
int mp_w4a16_linear_decode_host(const void* x_host_f16, void* x_stage_f16, const void* packed_i32,
                                const void* sz_f16x2, const void* bias_f16, void* y_stage_f16,
                                void* y_host_f16, int M, int N, int K, int group, mp_stream_t stream);
/* The same with a workspace of mp_w4a16_decode_workspace_bytes(M, N, K) bytes (zero-filled once, owned by the caller,
 * not shared between calls that may overlap): the kernel is then chosen as mp_w4a16_linear_decode chooses it. */
int mp_w4a16_linear_decode_host_ws(const void* x_host_f16, void* x_stage_f16, const void* packed_i32,
                                   const void* sz_f16x2, const void* bias_f16, void* y_stage_f16,
                                   void* y_host_f16, int M, int N, int K, int group, void* workspace,
                                   size_t workspace_bytes, mp_stream_t stream);
/*
 * Several independent host-buffer linears on one stream in one call (the q/k/v or gate/up projections of a
 * decoder layer, which read the same activations and do not depend on one another): all H2D copies are enqueued
 * first, then the kernels back to back -- so that, with mp_set_programmatic_launch(1), each one fetches its weights
 * while its predecessor drains -- then the D2H copies.  Every field means what the argument of the same name
 * means in mp_w4a16_linear_decode_host_ws; the entries must not share staging buffers or workspaces.  The call
 * stops at the first entry that fails and returns its status.
 */
typedef struct mp_host_linear {
  const void* x_host_f16;
  void* x_stage_f16;
  const void* packed_i32;
  const void* sz_f16x2;
  const void* bias_f16;
  void* y_stage_f16;
  void* y_host_f16;
  int M, N, K, group;
  void* workspace;
  size_t workspace_bytes;
} mp_host_linear;
int mp_w4a16_linear_decode_host_many(const mp_host_linear* linears, int count, mp_stream_t stream);
/*
 * The address under which the current device can read and write a page-locked
 * host range (cudaHostAlloc / cudaHostRegister memory, e.g. torch's pinned
 * tensors).  MP_ERR_UNSUPPORTED for pageable memory, a range that is not mapped
 * for this device or that spans two registrations.  No reference counterpart
 * (the reference's forward runs on host tensors directly).
 */
int mp_host_buffer_device_alias(const void* host_ptr, size_t bytes, void** device_ptr);

/*
 * Prefill variant (any M; meant for M > 64): the same linear on the fp16 tensor
 * cores (tcgen05 kind::f16, fp32 accumulators in TMEM), activations fed by TMA,
 * int4 unpack + group dequant fused in as a producer stage that writes the
 * dequantised tile straight into shared memory.  K % 64 == 0, group % 64 == 0.
 * error_word as for mp_w8a8_gemm.
 */
int mp_w4a16_linear_prefill(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                            const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                            int* error_word, mp_stream_t stream);
/*
 * Same, with scratch for split-K: with few output tiles (M <= 256 and a narrow
 * N) the K range of every tile is cut into slices so that all SMs stream
 * weights; the slices' fp32 partial tiles go to `workspace` and a second kernel
 * adds them in slice order (deterministic).  mp_w4a16_prefill_workspace_bytes
 * returns the size needed (0 = no split for this shape); a null workspace
 * means no split.
 */
size_t mp_w4a16_prefill_workspace_bytes(int M, int N, int K);
int mp_w4a16_linear_prefill_ex(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                               const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                               void* workspace, size_t workspace_bytes, int* error_word,
                               mp_stream_t stream);

/*
 * The workspace split-K decode linear for callers that cannot allocate device
 * memory.  (No counterpart in the reference; it exists for hosts of this
 * library -- a plugin inside another runtime's forward pass, code that runs
 * where cudaMalloc is off limits or under a frozen memory budget -- that have
 * no scratch buffer to hand in.)  Same arguments and results as
 * mp_w4a16_linear_decode minus the workspace: the split-K counters and partial
 * sums live in a fixed 8 MiB array inside the library, which every GPU that
 * loads the library holds until the process exits.  The call allocates
 * nothing.  Limits and rules:
 *   - M <= 64 as for the decode kernel; shapes whose partial sums do not fit
 *     the array (16 KiB + k_split * M * N * 4 bytes > 8 MiB, see
 *     mp_w4a16_linear_decode_static_max_bytes) return MP_ERR_WORKSPACE;
 *   - the first call on each device looks up the array's device address; make
 *     that first call before any stream capture;
 *   - all calls on a device share the array: two calls that can run at the
 *     same time on that device (different streams) race.  Calls ordered on
 *     one stream are fine; the counters are cleared at the start of each call.
 */
size_t mp_w4a16_linear_decode_static_max_bytes(void);
int mp_w4a16_linear_decode_static(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                                  const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                                  mp_stream_t stream);

/*
 * Programmatic dependent launch for the decode linears (default off; returns
 * the previous setting).  When on, a decode kernel may begin fetching its
 * WEIGHTS while the preceding kernel of the stream is still finishing;
 * activations, bias and outputs are only touched after that kernel has
 * completed.  Enable it only when no kernel still in flight writes the weight
 * buffers (weights are loaded once and then static, as in serving).
 * The same switch covers the W8A8 GEMMs and the kernels of the MoE layer
 * (routing, expert-parallel exchange and barriers, re-quantisation, combine):
 * each of them may be scheduled early, sets up its shared / tensor memory, and
 * then waits on the device for the preceding kernel before it reads or writes
 * anything else -- the launch latencies of the chain overlap, results are
 * the same bits.  The setting is read when a launch is issued (for a CUDA
 * graph: at capture).
 */
int mp_set_programmatic_launch(int enabled);

/*
 * The process-wide DEFAULT kernel behind the decode linears for M <= 16 (returns
 * the previous choice, or MP_ERR_INVALID_ARG); a call that must not depend on
 * what another host in the process has set passes its choice in the options of
 * mp_w4a16_linear_decode_opts instead.  Both compute F.linear(x, Wdq) of
 * awq/quantize/quantizer.py:109-130 with fp32 accumulation:
 *   MP_DECODE_KERNEL_UMMA      tcgen05.mma with the dequantised weights as the
 *                              tensor-memory operand (a thread expands one
 *                              weight row and stores it with tcgen05.st)
 *   MP_DECODE_KERNEL_MMA_SYNC  the mma.sync ring kernel (also the one behind
 *                              the row-parallel entry points)
 *   MP_DECODE_KERNEL_AUTO      (default) the tcgen05 kernel for 9..16 tokens on
 *                              weights of at least 40 MiB packed with at least
 *                              16384 output rows when a workspace was passed,
 *                              the mma.sync kernel otherwise
 * The tcgen05 kernel divides the (row block, K stage) pairs evenly over a
 * persistent grid and needs the workspace of mp_w4a16_decode_workspace_bytes
 * (zero-filled when created, left ready for the next call, not shared by calls
 * that overlap; re-zero it after a device-side wait has given up); without a
 * workspace, and for shapes the chosen kernel does not take, the call falls
 * through to the other kernels.
 */
#define MP_DECODE_KERNEL_MMA_SYNC 0
#define MP_DECODE_KERNEL_UMMA 1
#define MP_DECODE_KERNEL_AUTO 2
int mp_set_decode_kernel(int kind);
/* Which kernel (MP_DECODE_KERNEL_MMA_SYNC or _UMMA) the process default sends a decode call of this shape to
 * (1 <= M <= 64), with or without a workspace; shapes the chosen kernel does not take still fall through.  For
 * 17..64 rows _UMMA means the tcgen05 kernel with a 32- or 64-token activation tile (by default up to 32 rows
 * on >= 24 MiB of packed weights with >= 8192 output rows, up to 64 rows on >= 40 MiB with >= 16384), and
 * _MMA_SYNC that mp_w4a16_linear_decode would run its split-K kernel -- a caller then does better with
 * mp_w4a16_linear_prefill, the tensor-core GEMM. */
int mp_w4a16_decode_kernel_choice(int M, int N, int K, int have_workspace);

/*
 * mp_w4a16_linear_decode for M <= 64 with the kernel and programmatic dependent
 * launch chosen by THIS call (no process-wide state is read for what the
 * options name; 0 leaves everything at the process defaults):
 *   MP_DECODE_OPT_KERNEL_*     the kernel, as above.  For 17..64 rows
 *                              MP_DECODE_OPT_KERNEL_UMMA runs the tcgen05 kernel
 *                              with a 32- or 64-token activation tile (workspace
 *                              of mp_w4a16_decode_workspace_bytes); the other
 *                              choices run the workspace split-K kernel
 *   MP_DECODE_OPT_PDL_ON/_OFF  programmatic dependent launch for this call (see
 *                              mp_set_programmatic_launch for what it allows)
 */
#define MP_DECODE_OPT_KERNEL_MASK 0x7u
#define MP_DECODE_OPT_KERNEL_MMA_SYNC 0x1u
#define MP_DECODE_OPT_KERNEL_UMMA 0x2u
#define MP_DECODE_OPT_KERNEL_AUTO 0x4u
#define MP_DECODE_OPT_PDL_MASK 0x30u
#define MP_DECODE_OPT_PDL_ON 0x10u
#define MP_DECODE_OPT_PDL_OFF 0x20u
int mp_w4a16_linear_decode_opts(const void* x_f16, const void* packed_i32, const void* sz_f16x2,
                                const void* bias_f16, void* y_f16, int M, int N, int K, int group,
                                void* workspace, size_t workspace_bytes, unsigned int options,
                                mp_stream_t stream);

/*
 * Synchronously reads (and clears) the flag a decode kernel sets when one of
 * its bounded device-side waits gave up; *value == 0 means none did.  A
 * debugging aid: it synchronises with the device.
 */
int mp_read_decode_error(int* value);

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

/*
 * Residual add + RMSNorm + per-token int8 quantisation in one pass:
 *   residual <- f16(x + residual);  y = f16(f16(residual * rsqrt(mean(residual^2) + eps)) * gamma);
 *   (q, scale) = per-token absmax int8 of y (arithmetic of mp_act_quant_per_token).
 * Stands in for torch_npu.npu_add_rms_norm_dynamic_quant, whose (codes, scale)
 * pair the W8A8 linear takes as a tuple input
 * (acceleration/runtime_patches/vllm_ascend.patch:754-770, 3945-3962).  The
 * reference has no CPU statement of this fused op; the RMSNorm arithmetic is
 * that of the Hugging Face Llama RMSNorm the models use.  H % 8 == 0, H <= 16384.
 */
int mp_add_rmsnorm_quant(const void* x_f16, void* residual_f16, const void* gamma_f16, float eps, int M,
                         int H, void* q_i8, void* scale_f32, mp_stream_t stream);

/*
 * y[M,N] = f16( (qx[M,K] . w[N,K]^T as int32) * x_scale[m] * w_scale[n] (+ bias[n]) )
 * on the int8 tensor cores (tcgen05 kind::i8, int32 accumulators in TMEM).
 * Stands in for torch_npu.npu_quant_matmul as called by
 * AscendW8A8DynamicLinearMethod.apply
 * (acceleration/runtime_patches/vllm_ascend.patch:4007-4015), with the weight
 * kept in the reference's [out, in] layout.  Together with
 * mp_act_quant_per_token it is the real-int twin of SmoothQuantLinear.forward
 * (algorithm/quantization/ptq/smoothquant/source/smoothquant/fake_quant.py:84-88).
 * K % 16 == 0; all pointers 16-byte aligned.  error_word (device int, may be
 * NULL) is set to a non-zero value if a bounded device-side wait gives up.
 */
int mp_w8a8_gemm(const void* qx_i8, const void* x_scale_f32, const void* w_i8, const void* w_scale_f32,
                 const void* bias_f16, void* y_f16, int M, int N, int K, int* error_word,
                 mp_stream_t stream);
/*
 * Same, with scratch for split-K.  At decode and small-batch row counts the
 * GEMM is a weight stream over few output tiles; the K range of every tile is
 * then cut into slices so that all SMs stream weights, the slices' raw int32
 * partial tiles go to `workspace`, and a second kernel adds them (integer
 * sums: the split changes no output bit) and applies the scales.
 * mp_w8a8_gemm_workspace_bytes returns the size needed (0 = no split for this
 * shape); a null workspace means no split.
 */
size_t mp_w8a8_gemm_workspace_bytes(int M, int N, int K);
int mp_w8a8_gemm_ex(const void* qx_i8, const void* x_scale_f32, const void* w_i8,
                    const void* w_scale_f32, const void* bias_f16, void* y_f16, int M, int N, int K,
                    void* workspace, size_t workspace_bytes, int* error_word, mp_stream_t stream);

/*
 * Raw accumulators acc[M,N] = qx . w^T as int32: npu_quant_matmul with
 * output_dtype=int32 (acceleration/runtime_patches/vllm.patch:756-760), and
 * the bit-exact check of the tensor-core path.
 */
int mp_w8a8_gemm_i32(const void* qx_i8, const void* w_i8, void* acc_i32, int M, int N, int K,
                     int* error_word, mp_stream_t stream);

/*
 * OmniQuant-style W8A8: dynamic ASYMMETRIC 8-bit quantisation of each row (per token for
 * activations, per output channel for weights) to unsigned codes,
 *   s = clamp(f16(f16(max - min) / 255), 1e-5, 1e4), zp = rint(clamp(f16(-min / s), +-1e4)),
 *   u = clamp(f16(rint(f16(x / s)) + zp), 0, 255),
 * the arithmetic of UniformAffineQuantizer.per_token_dynamic_calibration + fake_quant
 * (algorithm/quantization/ptq/omniquant/source/omniquant/quantizer.py:124-150, 89-111).
 * Outputs: q_u8 [M,K], scale_f32 [M], zero_f32 [M] (integer valued), rowsum_i32 [M] = sum of the
 * row's codes; fake_f16 (optional) = f16(f16(u - zp) * s).  K % 8 == 0.
 */
int mp_affine_quant_per_row(const void* x_f16, int M, int K, void* q_u8, void* scale_f32, void* zero_f32,
                            void* rowsum_i32, void* fake_f16, mp_stream_t stream);

/*
 * y = f16( sum_k (qx - zx)(qw - zw) * sx[m] * sw[n] (+bias) ) with the sum evaluated exactly as
 * acc - zw*sum(qx) - zx*sum(qw) + K*zx*zw from a u8 x u8 -> int32 tensor-core product
 * (tcgen05 kind::i8, unsigned operands).  The real-int twin of QuantLinear.forward
 * (algorithm/quantization/ptq/omniquant/source/omniquant/int_linear.py:42-55).
 * K * 255 * 255 must fit int32 (K <= 33025).
 */
int mp_w8a8_affine_gemm(const void* qx_u8, const void* x_scale_f32, const void* x_zero_f32,
                        const void* x_rowsum_i32, const void* w_u8, const void* w_scale_f32,
                        const void* w_zero_f32, const void* w_rowsum_i32, const void* bias_f16,
                        void* y_f16, int M, int N, int K, int* error_word, mp_stream_t stream);

/* -------------------------------------------------------------------- MoE */

/*
 * Router: softmax over fp32 logits[T,E], top-k, renormalise, cast to f16 --
 * the in-repository statement of the Mixtral router,
 * FlatQuantMixtralSparseMoeBlock._route
 * (algorithm/quantization/qat/flatquant/source/flatquant/model_tools/mixtral_utils.py:330-333,349).
 * idx_i32 [T,k], weights_f16 [T,k].  k <= 8.
 */
int mp_moe_router_topk(const void* logits_f32, int T, int E, int k, void* idx_i32, void* weights_f16,
                       mp_stream_t stream);

/*
 * Sizes of the routing buffers for `max_rows` routed rows (T * k) over
 * `num_local_experts` experts: the number of ints in the plan, and the number
 * of rows of the expert-sorted buffers (every expert's segment is padded to a
 * multiple of 128 rows).
 */
size_t mp_moe_plan_ints(int num_local_experts, int max_rows);
int mp_moe_padded_rows(int num_local_experts, int max_rows);

/*
 * Routing + gather + per-token int8 quantisation for the experts
 * [expert_lo, expert_hi) this GPU owns: the role of
 * torch_npu.npu_moe_init_routing_quant in _run_expert_tile
 * (acceleration/runtime_patches/vllm_ascend.patch:2369-2379), i.e. lines
 * 174-183 of SmoothQuantPackedMoeExperts.forward (fake_quant.py).
 *   plan_i32          ints: counts[E] | cursors[E] | segment offsets[E+1] |
 *                     tile count | expert of each 128-row tile
 *   dest_row_i32      [T*k] row of entry (t,j) in the sorted buffers, -1 if
 *                     its expert is not local
 *   routed_q_i8       [padded_rows, H] int8 codes; routed_scale_f32 [padded_rows]
 * H % 16 == 0.
 */
int mp_moe_route_gather_quant(const void* hidden_f16, const void* topk_ids_i32, int T, int H, int k,
                              int expert_lo, int expert_hi, void* plan_i32, void* dest_row_i32,
                              void* routed_q_i8, void* routed_scale_f32, mp_stream_t stream);

/*
 * The expert MLP on routed, quantised rows: grouped int8 GEMM1 (gate|up) with
 * the SwiGLU epilogue, per-token re-quantisation, grouped int8 GEMM2 with the
 * dequant epilogue -- npu_grouped_matmul_swiglu_quant + npu_grouped_matmul of
 * _run_expert_tile (vllm_ascend.patch:2391-2412), i.e. fake_quant.py:184-187.
 *   w13_q_i8 [E, 2I, H] (gate rows first, then up), w13_scale_f32 [E, 2I]
 *   w2_q_i8  [E, H, I],                             w2_scale_f32  [E, H]
 *   d_out_f16 [padded_rows, H]
 */
size_t mp_moe_expert_stage_workspace_bytes(int padded_rows, int I);
int mp_moe_expert_stage(const void* routed_q_i8, const void* routed_scale_f32, const void* plan_i32,
                        int padded_rows, int H, int I, int num_local_experts,
                        const void* w13_q_i8, const void* w13_scale_f32, const void* w2_q_i8,
                        const void* w2_scale_f32, void* d_out_f16, void* workspace,
                        size_t workspace_bytes, int* error_word, mp_stream_t stream);
/*
 * Expert-parallel form of the stage: the second GEMM's epilogue stores every
 * result row straight into the result buffer of the rank the token came from
 * (peer stores over NVLink; peer_back_ptrs[s] = rank s's buffer [its routed
 * rows][H] fp16), located through the extended plan mp_moe_ep_plan wrote, so
 * there is no sorted result buffer and no separate return kernel.
 */
int mp_moe_expert_stage_scatter(const void* routed_q_i8, const void* routed_scale_f32,
                                const void* xplan_i32, int capacity_rows, int H, int I,
                                int num_local_experts, int world, const void* w13_q_i8,
                                const void* w13_scale_f32, const void* w2_q_i8, const void* w2_scale_f32,
                                void* const* peer_back_ptrs, void* workspace, size_t workspace_bytes,
                                int* error_word, mp_stream_t stream);

/*
 * Dense chunked gate/up projection with SwiGLU and per-token re-quantisation:
 * for every chunk c of the intermediate size,
 *   h_c = silu(x W_gate_c^T) * (x W_up_c^T),  (q_c, s_c) = int8 quant of h_c per token.
 * Replaces the reference's native op grouped_swiglu_loop_out
 * (acceleration/custom_ops/qwen2_5_vl/aclnn_grouped_swiglu_out_bridge.cpp:157-273;
 * its callers acceleration/runtime_patches/vllm.patch:114-170 and :959-1001),
 * which loops aclnnGroupedMatmulSwigluQuant over the chunks; here all chunks
 * are the groups of one grouped tcgen05 GEMM launch.
 *   x_i8        [T, H] int8 codes,       x_scale_f32 [T]
 *   w_i8        [chunks, 2C, H] int8: per chunk the C gate rows, then the C up
 *               rows (the reference's [1, H, 2C] per-chunk weight, transposed)
 *   w_scale_f32 [chunks, 2C]
 *   q_out_i8    [chunks, T, C],          scale_out_f32 [chunks, T]
 * Dequantisation, SiLU and the product round to fp16 as the expert path does
 * (smoothquant/fake_quant.py:184-186); scale = f16(max(|h|max, 1e-5) / 127).
 * H % 16 == 0, C % 16 == 0, chunks <= 256.
 */
size_t mp_w8a8_gate_up_swiglu_requant_workspace_bytes(int T, int H, int C, int chunks);
int mp_w8a8_gate_up_swiglu_requant(const void* x_i8, const void* x_scale_f32, const void* w_i8,
                                   const void* w_scale_f32, int T, int H, int C, int chunks,
                                   void* q_out_i8, void* scale_out_f32, void* workspace,
                                   size_t workspace_bytes, int* error_word, mp_stream_t stream);

/*
 * mp_moe_expert_stage in three launches (same workspace, same bits), each grouped GEMM optionally on ONE HALF of
 * the 256-row tiles in use (tile_part: -1 = all, 0 / 1 = first / second half; split at (tiles + 1) / 2).  An
 * expert-parallel caller uses the halves to overlap the exchange with the GEMMs on two streams -- the runtime's
 * own pattern of overlapping the token exchange with the expert matmuls
 * (acceleration/runtime_patches/vllm_ascend.patch:2482-2544):
 *   gemm1(0) | gemm1(1) | requant | gemm2(0) | gemm2(1)   on one stream,
 *   the pull of half 1 beside gemm1(0) and the push of half 0 beside gemm2(1) on another
 * (mp_moe_ep_pull_part / mp_moe_ep_push_part take the same `part`).  mp_moe_gemm1_swiglu(part 1) keeps the row
 * maxima part 0 produced; mp_moe_requant runs once, over all rows, between the two GEMMs.
 */
int mp_moe_gemm1_swiglu(const void* routed_q_i8, const void* routed_scale_f32, const void* plan_i32,
                        int padded_rows, int H, int I, int num_local_experts, const void* w13_q_i8,
                        const void* w13_scale_f32, void* workspace, size_t workspace_bytes, int tile_part,
                        int* error_word, mp_stream_t stream);
int mp_moe_requant(const void* plan_i32, int padded_rows, int I, int num_local_experts, void* workspace,
                   size_t workspace_bytes, mp_stream_t stream);
int mp_moe_gemm2(const void* plan_i32, int padded_rows, int I, int H, int num_local_experts,
                 const void* w2_q_i8, const void* w2_scale_f32, void* d_out_f16, void* workspace,
                 size_t workspace_bytes, int tile_part, int* error_word, mp_stream_t stream);

/*
 * out[t] = sum_j f16(d[dest_row(t,j)] * w[t,j]) in fp16, experts in ascending
 * order: npu_moe_token_unpermute (vllm_ascend.patch:2415-2419), i.e.
 * fake_quant.py:188-189.  Entries with dest_row < 0 are skipped.
 */
int mp_moe_combine(const void* d_f16, const void* dest_row_i32, const void* topk_ids_i32,
                   const void* topk_weights_f16, int T, int H, int k, void* out_f16, mp_stream_t stream);

/*
 * Expert-parallel exchange over peer-mapped (symmetric) memory, without a host
 * round trip -- the device-driven form of the runtime's all-to-all token
 * dispatcher / combiner (TokenDispatcherWithAll2AllV,
 * acceleration/runtime_patches/vllm_ascend.patch:3228-3236).  Every *_ptrs
 * argument is a host array of `world` device pointers, entry s being rank s's
 * buffer as mapped into this process (entry `rank` is the local buffer).
 *
 * mp_peer_barrier   cross-rank barrier on the stream: stores `epoch` (must grow by
 *                   one per call, same sequence on every rank) into slot `rank`
 *                   of every peer's flag array (uint32[world], zero at start) and
 *                   waits, for at most 2 s, until all local slots reached it; a
 *                   timeout sets *error_word = 4 and returns.
 * mp_peer_barrier_counted  the same barrier with the epoch kept in a device word
 *                   (zero at start) that the kernel advances itself, so that a
 *                   captured CUDA graph containing it can be replayed.
 * mp_moe_ep_plan    reads every peer's routing plan (as written by
 *                   mp_moe_route_gather_quant over all `num_experts` experts)
 *                   and lays out this rank's expert-sorted buffer: xplan_i32
 *                   (mp_moe_ep_plan_ints ints) starts with the plan
 *                   mp_moe_expert_stage takes.
 * mp_moe_ep_pull    copies the rows this rank's experts own out of the peers'
 *                   routed buffers (int8 rows + fp32 scales) into sorted order.
 * mp_moe_ep_push    stores each result row into its source rank's result buffer
 *                   at the row's original position.
 * capacity_rows: rows of the expert-sorted buffers (multiple of 256; an upper
 * bound, e.g. mp_moe_padded_rows(local experts, world * tokens * k)).
 */
int mp_peer_barrier(const void* const* peer_flag_ptrs, int world, int rank, unsigned int epoch,
                    int* error_word, mp_stream_t stream);
int mp_peer_barrier_counted(const void* const* peer_flag_ptrs, int world, int rank,
                            void* epoch_counter_u32, int* error_word, mp_stream_t stream);
/*
 * Row-parallel W8A8 linear (input features sharded over `world` GPUs) -- the role of
 * npu_mm_all_reduce_base(qx, W, hcom, reduce_op="sum", dequant_scale, pertoken_scale)
 * (acceleration/runtime_patches/vllm_ascend.patch:1428-1449): every rank quantises
 * its activation slice per token (mp_act_quant_per_token, scales into peer-mapped
 * memory), multiplies it with its weight slice into raw int32 accumulators in
 * peer-mapped memory (mp_w8a8_gemm_i32), then
 *   mp_peer_signal              advances the call counter (device word) and raises
 *                               it as this rank's arrival word on every peer;
 *   mp_w8a8_rowparallel_finish  waits (bounded, 2 s -> error word 5) for all arrival
 *                               words, reads every rank's accumulators and token
 *                               scales over NVLink and writes
 *                               f16(sum_r acc_r * xscale_r[m] * w_scale[n] (+bias)),
 *                               fp32 adds in rank order: the same bits on every rank.
 * Use two accumulator/scale buffers alternately (a peer may still read call n
 * while this rank computes call n+1).
 */
int mp_peer_signal(const void* const* peer_flag_ptrs, int world, int rank, void* epoch_counter_u32,
                   mp_stream_t stream);
int mp_w8a8_rowparallel_finish(const void* const* peer_acc_i32, const void* const* peer_xscale_f32,
                               const void* flags_u32, int world, const void* epoch_counter_u32, int M,
                               int N, const void* w_scale_f32, const void* bias_f16, void* y_f16,
                               int* error_word, mp_stream_t stream);
/*
 * mp_peer_publish                    copies up to two local ranges (A: 16-byte units, B: 4-byte units) to byte
 *                                    offsets offset_a / offset_b of this rank's receive slot -- slot0 or slot1 by
 *                                    the parity of the call number, which the kernel reads from epoch_counter_u32,
 *                                    advances and raises on every peer (block_counter: device int, zero between
 *                                    calls).  It replaces mp_peer_signal where the slot must alternate from call to
 *                                    call even inside a replayed CUDA graph: the producers write to ordinary local
 *                                    buffers and the slot is chosen on the device.
 * mp_w8a8_rowparallel_finish_parity  mp_w8a8_rowparallel_finish reading the slot of the call number's parity
 *                                    (entry [r] of the *0 / *1 arrays = rank r's slot 0 / slot 1).
 */
int mp_peer_publish(const void* src_a, int bytes_a, int offset_a, const void* src_b, int bytes_b, int offset_b,
                    void* slot0, void* slot1, void* const* peer_flags_u32, void* epoch_counter_u32,
                    int* block_counter, int world, int rank, mp_stream_t stream);
int mp_w8a8_rowparallel_finish_parity(const void* const* peer_acc0_i32, const void* const* peer_acc1_i32,
                                      const void* const* peer_xscale0_f32, const void* const* peer_xscale1_f32,
                                      const void* flags_u32, int world, const void* epoch_counter_u32, int M,
                                      int N, const void* w_scale_f32, const void* bias_f16, void* y_f16,
                                      int* error_word, mp_stream_t stream);

/*
 * All-gather of output slices for the column-parallel linear (output rows of the weight split over `world`
 * GPUs; the role of the runtime's tensor-parallel all-gather after a column-parallel linear,
 * acceleration/runtime_patches/vllm_ascend.patch:3260-3305): src [rows][slice_bytes] holds this rank's columns.
 * They are stored into every peer's receive buffer (peer_recv0 / peer_recv1, used alternately by call parity;
 * entry [r] = rank r's buffer, mp_peer_allgather_recv_bytes bytes each, zero before the first call) in a
 * flag-in-data form -- every 8 bytes on the wire are 4 bytes of payload and the call number -- so the receiver
 * polls the words it needs and neither a fence nor an arrival word is on the path; out [rows][world * slice_bytes]
 * receives this rank's slice directly and the peers' slices as they arrive (bounded wait, 2 s -> error word 7).
 * The call number lives in epoch_counter_u32 (device, zero at start; block_counter: device int, zero between
 * calls), so no argument changes between calls (graph-replayable).  slice_bytes % 16 == 0.
 */
size_t mp_peer_allgather_recv_bytes(int rows, int slice_bytes, int world);
int mp_peer_allgather_push(const void* src, int rows, int slice_bytes, void* const* peer_recv0,
                           void* const* peer_recv1, void* epoch_counter_u32, int* block_counter, int world,
                           int rank, void* out, int* error_word, mp_stream_t stream);

/*
 * Reduce-scatter + all-gather form of mp_w4a16_rowparallel_finish (the all-reduce after a row-parallel linear,
 * acceleration/runtime_patches/vllm_ascend.patch:3260-3305), for use after mp_w4a16_rowparallel_push on the same
 * stream: partial0_f32 / partial1_f32 are this rank's two partial-sum slots [M][N] (the push kernel wrote the
 * one of the call number's parity).  The columns rank q owns (N / world of them) are sent to q, which adds the
 * `world` partial sums in rank order (+ bias), rounds to fp16 and sends the result to everyone; both transfers use
 * the flag-in-data form of mp_peer_allgather_push (receive buffers peer_recv1_* of
 * mp_w4a16_rowparallel_recv_bytes(M_max, N, 1) bytes and peer_recv2_* of (M_max, N, 2) bytes, by call parity,
 * zero before the first call).  Every element is computed once, by its owner: identical bits on all ranks;
 * a rank sends 12 M N (world-1)/world bytes instead of reading 4 M N (world-1).  Bounded waits (2 s -> error
 * word 5).  N % (4 * world) == 0.
 */
size_t mp_w4a16_rowparallel_recv_bytes(int M, int N, int which);
int mp_w4a16_rowparallel_finish_ll(const void* partial0_f32, const void* partial1_f32,
                                   void* const* peer_recv1_0, void* const* peer_recv1_1,
                                   void* const* peer_recv2_0, void* const* peer_recv2_1, int world, int rank,
                                   const void* epoch_counter_u32, int M, int N, const void* bias_f16,
                                   void* y_f16, int* error_word, mp_stream_t stream);
/* mp_peer_barrier_counted followed by mp_moe_ep_plan in one launch (the block meets its peers, then reads their
 * counts): one kernel less on the path of every layer. */
int mp_moe_ep_barrier_plan(const void* const* peer_flag_ptrs, const void* const* peer_plan_ptrs, int world, int rank,
                           void* epoch_counter_u32, int num_experts, int capacity_rows, void* xplan_i32,
                           int* error_word, mp_stream_t stream);
size_t mp_moe_ep_plan_ints(int world, int num_local_experts, int capacity_rows);
int mp_moe_ep_plan(const void* const* peer_plan_ptrs, int world, int rank, int num_experts,
                   int capacity_rows, void* xplan_i32, mp_stream_t stream);
int mp_moe_ep_pull(const void* const* peer_q_ptrs, const void* const* peer_scale_ptrs, const void* xplan_i32,
                   int world, int num_local_experts, int capacity_rows, int H, void* q_sorted_i8,
                   void* scale_sorted_f32, mp_stream_t stream);
int mp_moe_ep_push(const void* d_sorted_f16, const void* xplan_i32, int world, int num_local_experts,
                   int capacity_rows, int H, const void* const* peer_back_ptrs, mp_stream_t stream);
/* The same two copies restricted to one half of the 256-row tiles in use (part 0 / 1; -1 = all rows), split where
 * mp_moe_gemm1_swiglu / mp_moe_gemm2 split their tiles. */
int mp_moe_ep_pull_part(const void* const* peer_q_ptrs, const void* const* peer_scale_ptrs, const void* xplan_i32,
                        int world, int num_local_experts, int capacity_rows, int H, void* q_sorted_i8,
                        void* scale_sorted_f32, int part, mp_stream_t stream);
int mp_moe_ep_push_part(const void* d_sorted_f16, const void* xplan_i32, int world, int num_local_experts,
                        int capacity_rows, int H, const void* const* peer_back_ptrs, int part, mp_stream_t stream);
/*
 * The return path with the closing barrier folded into its two neighbours (two launches instead of three).
 * mp_moe_ep_push_signal = mp_moe_ep_push, after which the block that finishes last advances *epoch_counter_u32 and
 * raises this rank's arrival word on every peer (peer_flag_ptrs as for mp_peer_barrier_counted; block_counter_i32
 * is a device int that is zero between calls).  mp_moe_combine_after_peers = mp_moe_combine whose blocks first
 * wait (bounded, 2 s -> error word 4) until every peer's arrival word in this rank's own array has reached
 * *epoch_counter_u32, i.e. until all result rows have landed in d_f16.  Both calls go on the same stream, the push
 * first; every rank issues the same sequence of epoch-advancing calls.
 */
int mp_moe_ep_push_signal(const void* d_sorted_f16, const void* xplan_i32, int world, int num_local_experts,
                          int capacity_rows, int H, const void* const* peer_back_ptrs,
                          const void* const* peer_flag_ptrs, int rank, void* epoch_counter_u32,
                          void* block_counter_i32, mp_stream_t stream);
int mp_moe_combine_after_peers(const void* arrival_words_u32, int world, const void* epoch_counter_u32,
                               const void* d_f16, const void* dest_row_i32, const void* topk_ids_i32,
                               const void* topk_weights_f16, int T, int H, int k, void* out_f16,
                               int* error_word, mp_stream_t stream);

/*
 * dst row i = src row row_map[i] (rows of row_bytes bytes; 4, or a multiple of
 * 16); a negative map entry gives a zero row.  The row permutation an
 * expert-parallel rank applies to what its peers sent (source-major) to get
 * expert-sorted rows, and back -- the re-ordering torch_npu.npu_moe_init_routing_v2
 * performs with active_expert_range after an all-gather dispatch
 * (acceleration/runtime_patches/vllm_ascend.patch:3158-3214).
 */
int mp_gather_rows(const void* src, const void* row_map_i32, int n_dst_rows, int row_bytes, void* dst,
                   mp_stream_t stream);

#ifdef __cplusplus
}
#endif
#endif /* MINDPIPE_B200_H_ */
