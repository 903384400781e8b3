/*
 * rexsc_b200.h -- C ABI of the B200 (sm_100a) implementation of the REX-SC stochastic-computing
 * arithmetic: LFSR bit-stream generation, SC conv2d / linear forward with OR-n accumulation,
 * the point-wise OR-n / calibration / error-injection kernels and the FXP saturating conv.
 *
 * Conventions
 *   - every pointer named d_* is a DEVICE pointer on the current CUDA device;
 *   - `stream` is a cudaStream_t passed as void*; all work is enqueued on it, nothing synchronises;
 *   - functions return REXSC_OK (0) or a negative REXSC_E_* code and never throw;
 *   - no allocation and no numeric state kept between calls: scratch is a caller-owned workspace whose size
 *     the matching *_workspace_size() function reports (the reference keeps ~1.3 GiB of process-lifetime
 *     scratch instead: torch_c/sc-extension/sc_cuda_kernel.cu:622-632, sc_device.cuh:711-714).  The only
 *     library-owned device memory is the fixed array behind rexsc_sc_conv2d_fwd_static; the only host-side
 *     state is a per-thread cache of derived launch plans (pure functions of the descriptors) and the text
 *     of the last CUDA error;
 *   - int16 outputs of the SC conv must be at least 4-byte aligned (16-byte aligned outputs take the
 *     vectorised store path); tensors from an allocator always are, offset views may not be;
 *   - each entry point cites the reference interface it replaces (paths inside nanocad-lab/rex-sc).
 */
#ifndef REXSC_B200_H
#define REXSC_B200_H

#include <stddef.h>
#include <stdint.h>

#ifdef __cplusplus
extern "C" {
#endif

#define REXSC_ABI_VERSION 1

enum {
    REXSC_OK = 0,
    REXSC_E_BAD_ARG = -1,       /* null pointer, non-positive size, unknown enum value                  */
    REXSC_E_UNSUPPORTED = -2,   /* valid in the reference but outside what this library implements      */
    REXSC_E_WORKSPACE = -3,     /* workspace pointer null, misaligned or smaller than *_workspace_size  */
    REXSC_E_TOO_LONG = -4,      /* dot product / stream longer than the accumulators can count          */
    REXSC_E_CUDA = -5,          /* a CUDA runtime call or launch failed (see rexsc_last_cuda_error)     */
    REXSC_E_DEVICE_TIMEOUT = -6, /* a bounded device-side wait gave up (reported by rexsc_workspace_status) */
    REXSC_E_STATIC_SCRATCH = -7  /* the call needs more scratch than the library's built-in array holds      */
};

enum { REXSC_F32 = 0, REXSC_F16 = 1, REXSC_BF16 = 2 };

/* Which SC conv kernel to use; all give identical results.  DIRECT: one thread per output, any shape and any n.
 * TILED: shared-memory implicit GEMM on the integer ALU pipe (LOP3 thermometers).  TENSOR: one int8 tcgen05 GEMM
 * per time slot with min(count, n) applied to the TMEM accumulators (filters of at most 9 taps, any stride whose
 * residue planes fit its shared-memory patch).  AUTO picks TENSOR whenever the shape fits it and there are at least
 * 32 input channels, else TILED when the shape fits that, else DIRECT. */
enum { REXSC_KERNEL_AUTO = 0, REXSC_KERNEL_DIRECT = 1, REXSC_KERNEL_TILED = 2, REXSC_KERNEL_TENSOR = 3 };

/*
 * Shape / configuration of one SC conv2d (or, with h = w = kh = kw = 1, SC linear) forward.
 * Field meanings follow the argument list of conv2d_generic_general_split_acc
 * (torch_c/sc-extension/sc_cuda.cpp:87, bound at :124) so that a binding can fill it 1:1.
 */
typedef struct rexsc_sc_conv_desc {
    int32_t batch, c_in, h_in, w_in; /* activation, logical NCHW extents before the op's own padding  */
    int32_t c_out, kh, kw;           /* weight [c_out][c_in][kh][kw]                                   */
    int32_t pad_h, pad_w;            /* zero padding added by the op (reference: padding[1], padding[0]) */
    int32_t stride_h, stride_w;      /* reference: stride[0] on dim 2, stride[1] on dim 3              */
    int32_t act_dtype, act_channels_last;  /* REXSC_F32/F16/BF16; 1 = dense NHWC memory, 0 = dense NCHW */
    int32_t w_dtype, w_channels_last;      /* same for the weight (OHWI vs OIHW)                        */
    int32_t out_channels_last;       /* memory format of the int16 outputs (reference: = activation's) */
    int32_t bit_length;              /* stream length L                                                */
    int32_t lfsr_length;             /* < 0: derived from bit_length as the reference does             */
    int32_t bin_config;              /* OR-n with n = bin_config + 1; n >= dot-product length = plain count */
    int32_t gen_config;              /* AND-g generator replication, 1 in every reference configuration */
    int32_t xnor;                    /* XNOR-feedback LFSR and seed offset (conv only)                  */
    int32_t prog_total_width, prog_load_width, prog_load_wait; /* progressive loading (7, 8, 1 = off)  */
    int32_t linear_seeds;            /* 1: seeds depend on c_in only and xnor is ignored (SC linear)   */
    int32_t kernel;                  /* REXSC_KERNEL_*                                                 */
} rexsc_sc_conv_desc;

/* Library identification. */
int rexsc_abi_version(void);
/* Text of the last CUDA error seen by this library on the calling thread ("" if none). */
const char *rexsc_last_cuda_error(void);
/* Kernels this library has launched in the calling process so far, on any device and stream (memsets and copies are
 * not kernels).  The difference between two reads counts the launches of the calls in between. */
unsigned long long rexsc_kernel_launch_count(void);

/*
 * SC conv2d forward.  Replaces conv2d_generic_general_split_acc / conv2d_generic_general_acc
 * (torch_c/sc-extension/sc_cuda.cpp:73-99) and everything below them:
 * conv2d_generic_cuda_general_gemm (sc_cuda_kernel.cu:565-757), the stream generators
 * (sc_cuda_conv.cu:3-166), im2col / GEMM / scatter kernels (sc_cuda_kernel.cu:367-562,
 * sc_device.cu:186-386).  Pad + quantise + stream generation + OR-n accumulation in one call.
 *   d_act     activation, dtype/layout per desc, [batch][c_in][h_in][w_in] logical
 *   d_weight  weight, dtype/layout per desc
 *   d_out_pos, d_out_neg  int16 [batch][c_out][oh][ow] in the layout desc->out_channels_last names;
 *             either may alias nothing else; both are fully overwritten
 */
size_t rexsc_sc_conv2d_workspace_size(const rexsc_sc_conv_desc *desc);
/* Which kernel a forward call with this descriptor runs: REXSC_KERNEL_DIRECT, _TILED or _TENSOR, or a negative
 * REXSC_E_* code (REXSC_E_UNSUPPORTED when desc->kernel forces a kernel the shape does not fit, e.g. a patch
 * larger than the tiled kernel's shared-memory stage).  Host-only, launches nothing. */
int rexsc_sc_conv2d_kernel_choice(const rexsc_sc_conv_desc *desc);
int rexsc_sc_conv2d_fwd(const rexsc_sc_conv_desc *desc, const void *d_act, const void *d_weight,
                        int16_t *d_out_pos, int16_t *d_out_neg, void *d_workspace, size_t workspace_bytes,
                        void *stream);

/*
 * SC conv2d forward without a caller workspace and without any allocation.  No counterpart in the reference
 * (its kernels cudaMalloc their scratch on first use, torch_c/sc-extension/sc_cuda_kernel.cu:622-632).
 * Meant for callers that cannot allocate device memory: a plugin inside an application whose own pool owns
 * the device memory, or a loop that bans allocation calls once it is running because they synchronise the
 * device.  Same arguments and bit-identical results as rexsc_sc_conv2d_fwd, with the scratch taken from a
 * fixed 32 MiB array inside the library (rexsc_sc_conv2d_static_scratch_bytes), which every GPU that loads
 * the library holds until the process ends.  Returns REXSC_E_STATIC_SCRATCH, launching nothing, when
 * rexsc_sc_conv2d_workspace_size(desc) is larger than that.  Every call asks the runtime for the array's device
 * address (no allocation; still valid after a device reset); the first call on a device may load the library's
 * module there: make it before any stream capture starts.  All calls share the array (each call rewrites
 * what it reads and clears its status word), so calls that overlap on the GPU race: serialise them.
 * rexsc_sc_conv2d_static_status(stream) is the twin of rexsc_workspace_status for this array: it synchronises the
 * stream and returns REXSC_OK, or REXSC_E_DEVICE_TIMEOUT when a bounded device-side wait of the last call gave up
 * (its outputs are then incomplete).  It allocates nothing either.
 */
size_t rexsc_sc_conv2d_static_scratch_bytes(void);
int rexsc_sc_conv2d_fwd_static(const rexsc_sc_conv_desc *desc, const void *d_act, const void *d_weight,
                               int16_t *d_out_pos, int16_t *d_out_neg, void *stream);
int rexsc_sc_conv2d_static_status(void *stream);

/*
 * The two stages of rexsc_sc_conv2d_fwd as separate calls (same descriptor, same workspace):
 *   expand      pad + quantise + stream generation of activations and weights into the workspace
 *               (replaces the reference's K1/K2 generators, sc_cuda_conv.cu:3-166, and the libtorch
 *               quantisation passes of sc_cuda.cpp:88-94);
 *   accumulate  OR-n accumulation of the stream words into the int16 outputs (replaces im2col + GEMM +
 *               scatter, sc_cuda_kernel.cu:367-562 and sc_device.cu:186-386).
 * fwd == expand followed by accumulate on the same stream.  Splitting lets a caller time the stages or keep
 * expanded streams across calls while the tensors they came from are unchanged: expand accepts a null d_act or a
 * null d_weight (not both) and then leaves that operand's part of the workspace as an earlier expand with the same
 * descriptor wrote it -- e.g. inference expands the weights of a layer once and only the activations per call.
 * The workspace also records HOW the last activation expand laid the activations out (3x3 stride-1 layers drop the
 * zero border from their bit planes when the border is indeed zero, which the expand stage checks on the device), so
 * accumulate must be given the descriptor and workspace of the activation expand that precedes it on the stream.
 * Between the kernels of one call the device decides which of two prepared launches runs; nothing synchronises
 * with the host.
 */
int rexsc_sc_conv2d_expand(const rexsc_sc_conv_desc *desc, const void *d_act, const void *d_weight,
                           void *d_workspace, size_t workspace_bytes, void *stream);
int rexsc_sc_conv2d_accumulate(const rexsc_sc_conv_desc *desc, int16_t *d_out_pos, int16_t *d_out_neg,
                               void *d_workspace, size_t workspace_bytes, void *stream);

/*
 * SC linear forward.  Replaces linear_generic_general_acc (torch_c/sc-extension/sc_cuda.cpp:101-120)
 * and linear_generic_cuda_general (sc_cuda_matmul.cu:584-747).  A convenience over the conv entry
 * point: d_act is [batch][c_in], d_weight [c_out][c_in], outputs int16 [batch][c_out]; seeds depend
 * on c_in only and the XOR LFSR is always used, as in the reference.
 */
size_t rexsc_sc_linear_workspace_size(int32_t batch, int32_t c_in, int32_t c_out, int32_t bit_length,
                                      int32_t lfsr_length, int32_t gen_config);
int rexsc_sc_linear_fwd(int32_t batch, int32_t c_in, int32_t c_out, int32_t act_dtype, int32_t w_dtype,
                        int32_t bit_length, int32_t lfsr_length, int32_t bin_config, int32_t gen_config,
                        int32_t prog_total_width, int32_t prog_load_width, int32_t prog_load_wait,
                        const void *d_act, const void *d_weight, int16_t *d_out_pos, int16_t *d_out_neg,
                        void *d_workspace, size_t workspace_bytes, void *stream);

/*
 * The same op with the seed offsets of the weight generators as arguments: the stream of weight (co, c) starts from
 * LFSR state (offset + c) mod (2^l - 1) + 1, offset = w_seed_pos for a positive and w_seed_neg for a negative weight.
 * rexsc_sc_linear_fwd is the (13, 13) of the extension (sc_cuda_matmul.cu:77-78).  (67, 37) with OR-1 (bin_config 0)
 * or plain counting reproduces the per-bit torch loop of the reference's linear_generic with generator='lfsr' and
 * shared generators (utils_functional.py:147-165, 1016-1036): pos / bit_length and neg / bit_length are its
 * result_pos.mean(0) and result_neg.mean(0).  Offsets must not be negative.
 */
int rexsc_sc_linear_fwd_seeded(int32_t batch, int32_t c_in, int32_t c_out, int32_t act_dtype, int32_t w_dtype,
                               int32_t bit_length, int32_t lfsr_length, int32_t bin_config, int32_t gen_config,
                               int32_t prog_total_width, int32_t prog_load_width, int32_t prog_load_wait,
                               int32_t w_seed_pos, int32_t w_seed_neg, const void *d_act, const void *d_weight,
                               int16_t *d_out_pos, int16_t *d_out_neg, void *d_workspace, size_t workspace_bytes,
                               void *stream);

/*
 * Reads the device status word of a workspace used by the call(s) above: synchronises `stream`,
 * returns REXSC_OK or REXSC_E_DEVICE_TIMEOUT.  Optional (debug / tests); the forward calls
 * themselves never synchronise.
 */
int rexsc_workspace_status(const void *d_workspace, void *stream);

/*
 * Stream words of the LFSR/comparator generator, for inspection and tests: fills
 * d_lut[(phase * (1 << l) + value) * words + j] with bits 32j..32j+31 of the stream of an element
 * whose seed index is congruent to `phase` modulo 2^l - 1 (bit t = time slot t).
 * Restates the generation loops of torch_c/sc-extension/sc_cuda_conv.cu:70-92,149-163 and the
 * LFSR formulas of sc_device.cuh:108-286.  words = ceil(bit_length * gen_config / 32).
 */
int rexsc_build_lfsr_lut(int32_t lfsr_length, int32_t bit_length, int32_t gen_config, int32_t xnor,
                         int32_t prog_total_width, int32_t prog_load_width, int32_t prog_load_wait,
                         int32_t is_weight, uint32_t *d_lut, void *stream);

/*
 * Point-wise OR-n activation.  Replaces or_approx_n_forward_acc / or_approx_n_backward_acc
 * (torch_c/sc-extension/sc_cuda_pw.cu:708-746,767-811; kernels :15-69,86-144; scalar math
 * sc_device.cuh:393-430,466-505).  or_n in 1..4.  Tensors are flat dense buffers of n_elem elements.
 *   fwd: out_f32[i] = f_n(in[i])
 *   bwd: grad_in_f32[i] = grad_out_f32[i] * f_n'(half(in[i]))   (the reference rounds the saved sum to fp16)
 */
int rexsc_orn_fwd(const void *d_in, int32_t in_dtype, float *d_out, int64_t n_elem, int32_t or_n, void *stream);
int rexsc_orn_bwd(const float *d_grad_out, const void *d_in, int32_t in_dtype, float *d_grad_in,
                  int64_t n_elem, int32_t or_n, void *stream);

/*
 * Fused OR-n(pos) - OR-n(neg) with 5th-order bias polynomial and std-polynomial * N(0,1) injection.
 * Replaces or_approx_n_forward_bias_std_both_acc / or_approx_n_backward_bias_std_both_acc
 * (torch_c/sc-extension/sc_cuda_pw.cu:863-927,952-1011; kernels :219-373,527-621; scalar math
 * sc_device.cuh:507-657).  d_bias_coef / d_std_coef: fp32 device arrays with at least 6 entries.
 * Noise: counter-based Philox4x32-10 keyed by `seed`, counter = (element index / 4, `offset`, sign);
 * the caller advances `offset` per call (the reference keeps 320000 persistent cuRAND states instead,
 * sc_cuda_pw.cu:699-706,878-882).  With all std coefficients zero the result does not depend on the noise.
 */
int rexsc_orn_bias_std_both_fwd(const void *d_pos, const void *d_neg, int32_t in_dtype, const float *d_bias_coef,
                                const float *d_std_coef, float *d_out, int64_t n_elem, int32_t or_n,
                                uint64_t seed, uint64_t offset, void *stream);
int rexsc_orn_bias_std_both_bwd(const float *d_grad_out, const void *d_pos, const void *d_neg, int32_t in_dtype,
                                const float *d_bias_coef, float *d_grad_pos, float *d_grad_neg, int64_t n_elem,
                                int32_t or_n, void *stream);

/*
 * Single-sided variants.  Replace or_approx_n_forward_bias_std_acc / or_approx_n_backward_bias_std_acc
 * (torch_c/sc-extension/sc_cuda_pw.cu:834-861,929-950; kernels :375-418,493-525).  The forward rounds
 * its input to fp16 and returns fp16, as the reference does.
 */
int rexsc_orn_bias_std_fwd(const void *d_in, int32_t in_dtype, const float *d_bias_coef, const float *d_std_coef,
                           void *d_out_f16, int64_t n_elem, int32_t or_n, uint64_t seed, uint64_t offset,
                           void *stream);
int rexsc_orn_bias_std_bwd(const float *d_grad_out, const void *d_in, int32_t in_dtype, const float *d_bias_coef,
                           float *d_grad_in, int64_t n_elem, int32_t or_n, void *stream);

/*
 * Caller arithmetic on the SC conv's int16 counts, one pass instead of five.  Replaces, in the caller of
 * conv2d_generic_general_split_acc, `result_pos.to(dtype)`, `result_neg.to(dtype)` (utils_functional.py:1181-1182),
 * `result_pos / bit_length`, `result_neg / bit_length` (:1273-1274) and `result_pos_value - result_neg_value`
 * (:1324).  out_dtype REXSC_F32 or REXSC_F16 (the dtype under autocast); bit_length must be a power of two, which
 * makes every scaling exact, so the outputs equal the eager sequence bit for bit (fp16 rounds counts above 2048 and
 * the difference, as eager does).  Any of the three outputs may be null, not all:
 *   val_pos[i] = dtype(pos[i]) / L     val_neg[i] = dtype(neg[i]) / L     val_diff[i] = val_pos[i] - val_neg[i]
 */
int rexsc_sc_counts_to_value(const int16_t *d_pos, const int16_t *d_neg, int32_t bit_length, int32_t out_dtype,
                             void *d_val_pos, void *d_val_neg, void *d_val_diff, int64_t n_elem, void *stream);

/*
 * Calibration statistics on the device.  Replaces the 30 masked mean / std passes of compute_bias_std_coef
 * (utils_functional.py:901-925) over a_bit = cat(pos, neg) / L and a_act = cat(guide_pos, guide_neg): for each of the
 * 30 windows [e_i, e_i + 0.1) of the guide value, e = numpy.linspace(0, max(a_bit), 30) rounded to fp32 as the
 * tensor comparison does, the number of elements, the sum of err = a_bit - a_act (fp32) and the sum of err^2.
 * The least-squares fit of the two 5th-order polynomials stays with the caller.  Three launches (clear, maximum,
 * windows), no host synchronisation, d_stats is the only memory written:
 *   double sums[30][3]  {count, sum err, sum err^2} per window     (offset 0)
 *   int32  max_count    largest count of either sign               (offset 720)
 *   int32  reserved
 * d_stats: REXSC_CALIB_STATS_BYTES of device memory, 8-byte aligned.  guide_dtype REXSC_F32 or REXSC_F16.
 * counts_via_half != 0 rounds each count to fp16 first, as `.to(float16)` under autocast does (exact up to 2048).
 * REXSC_F16 guide values are widened to fp32 before the comparisons and the subtraction, i.e. the result equals
 * compute_bias_std_coef(a_bit, a_act.float()); torch itself would round the window edges and err to fp16 for a half
 * a_act.  The reference's front end never has a half a_act (its guide values are the fp32 outputs of
 * or_approx_n_forward_acc, utils_functional.py:474,1234-1235); REXSC_F32 with counts_via_half is its autocast case.
 */
#define REXSC_CALIB_BINS 30
#define REXSC_CALIB_STATS_BYTES (REXSC_CALIB_BINS * 3 * 8 + 8)
int rexsc_sc_calib_stats(const int16_t *d_pos, const int16_t *d_neg, const void *d_guide_pos, const void *d_guide_neg,
                         int32_t guide_dtype, int32_t bit_length, int32_t counts_via_half, int64_t n_elem,
                         void *d_stats, void *stream);
/*
 * The two stages of rexsc_sc_calib_stats as separate calls, for callers that calibrate over a batch sharded across
 * GPUs (the reference calibrates on one GPU's batch, utils_functional.py:1290-1298; no counterpart there):
 *   max      clears d_stats and writes the largest count of this shard into max_count;
 *   windows  reads max_count from d_stats and ADDS this shard's window sums to sums[][].
 * Between the two, a data-parallel caller all-reduces max_count (MAX) so that every rank uses the same windows; after
 * windows it all-reduces sums (SUM): every rank then fits the same polynomials, those of the global batch.
 * stats == max followed by windows on the same stream.
 */
int rexsc_sc_calib_max(const int16_t *d_pos, const int16_t *d_neg, int32_t bit_length, int64_t n_elem, void *d_stats,
                       void *stream);
int rexsc_sc_calib_windows(const int16_t *d_pos, const int16_t *d_neg, const void *d_guide_pos,
                           const void *d_guide_neg, int32_t guide_dtype, int32_t bit_length, int32_t counts_via_half,
                           int64_t n_elem, void *d_stats, void *stream);

/*
 * FXP fixed-point conv with saturating accumulation.  Replaces conv2d_saturate_acc
 * (torch_c/sc-extension/fixed_cuda.cpp:24-34) and conv2d_saturate_cuda / compute_saturate_general
 * (fixed_cuda_kernel.cu:82-347).  Pad + quantise (round-half-even) + saturating accumulate.
 * Activation and weight are dense NCHW / OIHW (the reference kernel indexes NCHW only,
 * fixed_cuda_kernel.cu:125,179-182); output int32 NCHW [batch][c_out][oh][ow].
 */
typedef struct rexsc_fxp_conv_desc {
    int32_t batch, c_in, h_in, w_in;
    int32_t c_out, kh, kw;
    int32_t pad_h, pad_w, stride_h, stride_w;
    int32_t act_dtype, w_dtype;
    int32_t add_config;    /* 0 fixed-point add, 1 simulated OR add, >= 2 simulated OR-2 pairs */
    int32_t precision_in;  /* quantisation scale 2^precision_in                                */
    int32_t precision_out; /* accumulator precision                                            */
    int32_t kernel;        /* 0 auto, 1 CUDA-core kernels only, 2 tensor-core (tcgen05 int8) closed form,
                              3 the same with unswizzled shared-memory operand tiles               */
} rexsc_fxp_conv_desc;
size_t rexsc_fxp_conv2d_workspace_size(const rexsc_fxp_conv_desc *desc);
int rexsc_fxp_conv2d_fwd(const rexsc_fxp_conv_desc *desc, const void *d_act, const void *d_weight,
                         int32_t *d_out, void *d_workspace, size_t workspace_bytes, void *stream);

/*
 * Register-only LOP3 issue-rate probe used by the benchmark to measure the integer-ALU roofline the
 * SC conv kernels are measured against.  Launches `blocks` x 256 threads doing `iters` x 64 dependent-free
 * LOP3 per thread; d_sink receives one word per thread.  Total lane-ops = blocks*256*iters*64.
 */
int rexsc_alu_probe(int32_t blocks, int32_t iters, uint32_t *d_sink, void *stream);

/*
 * Tensor-pipe probe used by the benchmark to measure the int8 tcgen05 rate the tensor-core SC conv kernel is measured
 * against: `blocks` CTAs (two fit an SM) each issue iters x 16 int8 MMAs of shape M128 x n_cols x K32 (n_cols 128
 * or 256) on fixed shared-memory operands.  Total multiply-accumulates = blocks*iters*16*128*n_cols*32.
 * d_sink receives blocks*128 words.
 */
int rexsc_mma_probe(int32_t blocks, int32_t iters, int32_t n_cols, uint32_t *d_sink, void *stream);

#ifdef __cplusplus
}
#endif
#endif /* REXSC_B200_H */
