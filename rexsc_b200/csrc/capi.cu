// extern "C" entry points of the SC conv / linear forward, plus library-wide helpers.
#include <atomic>
#include <stdio.h>
#include <string.h>

#include "common.cuh"

namespace rexsc {

static thread_local char g_cuda_error[256] = "";

void set_cuda_error(cudaError_t e, const char *where)
{
    snprintf(g_cuda_error, sizeof(g_cuda_error), "%s: %s (%s)", where, cudaGetErrorName(e), cudaGetErrorString(e));
}

static std::atomic<unsigned long long> g_kernel_launches{0};

void note_kernel_launch() { g_kernel_launches.fetch_add(1, std::memory_order_relaxed); }

struct ConvBuffers {
    int *status;
    uint32_t *lut_a, *lut_w, *A, *Wt, *S;
    void *tc;
};

// which accumulate kernel a descriptor resolves to (or a negative error)
static int resolve_kernel(const rexsc_sc_conv_desc *desc, const ConvPlan &p)
{
    const bool tiled_ok = conv_tiled_supported(p);
    switch (desc->kernel) {
    case REXSC_KERNEL_DIRECT: return REXSC_KERNEL_DIRECT;
    case REXSC_KERNEL_TILED: return tiled_ok ? (int)REXSC_KERNEL_TILED : (int)REXSC_E_UNSUPPORTED;
    case REXSC_KERNEL_TENSOR: return p.tc_ok ? (int)REXSC_KERNEL_TENSOR : (int)REXSC_E_UNSUPPORTED;
    default:
        // AUTO: the tensor-core kernel wherever it fits (up to 9 taps, any stride) and the dot product fills its
        // 32-channel K words; thin inputs and large filters keep the ALU kernels.
        if (p.tc_ok && p.C >= 32) return REXSC_KERNEL_TENSOR;
        return tiled_ok ? (int)REXSC_KERNEL_TILED : (int)REXSC_KERNEL_DIRECT;
    }
}

static int conv_buffers(const rexsc_sc_conv_desc *desc, void *d_workspace, size_t workspace_bytes, ConvPlan *p,
                        ConvBuffers *b)
{
    int rc = make_conv_plan(desc, p);
    if (rc != REXSC_OK) return rc;
    if (desc->kernel < REXSC_KERNEL_AUTO || desc->kernel > REXSC_KERNEL_TENSOR) return REXSC_E_BAD_ARG;
    if (!d_workspace || workspace_bytes < p->total || (reinterpret_cast<uintptr_t>(d_workspace) & 255))
        return REXSC_E_WORKSPACE;
    uint8_t *ws = static_cast<uint8_t *>(d_workspace);
    b->status = reinterpret_cast<int *>(ws + p->off_status);
    b->lut_a = reinterpret_cast<uint32_t *>(ws + p->off_lut_a);
    b->lut_w = reinterpret_cast<uint32_t *>(ws + p->off_lut_w);
    b->A = reinterpret_cast<uint32_t *>(ws + p->off_A);
    b->Wt = reinterpret_cast<uint32_t *>(ws + p->off_Wt);
    b->S = reinterpret_cast<uint32_t *>(ws + p->off_S);
    b->tc = ws + p->off_tc;
    return REXSC_OK;
}

// Activation grid of the tensor-core path for a plan (see make_compact_plan in common.cuh):
//   kGridStandard     every padded pixel is stored;
//   kGridCompact      the compact grid, valid by construction: the descriptor itself pads by at least one pixel;
//   kGridSpeculative  the layer qualifies but the border is the caller's data (a caller that pads before the call, as
//                     the reference's front end does): the expand stage checks the border on the device and leaves
//                     its verdict in word 1 of the status block (0: compact planes, 1: standard planes), and the
//                     accumulate stage launches one kernel for either outcome, of which the verdict lets one run.
enum { kGridStandard = 0, kGridCompact = 1, kGridSpeculative = 2 };

static int grid_mode(const rexsc_sc_conv_desc *desc, const ConvPlan &p, int kernel, ConvPlan *pc)
{
    if (kernel != REXSC_KERNEL_TENSOR || desc->linear_seeds || !make_compact_plan(p, pc)) return kGridStandard;
    return (p.ph >= 1 && p.pw >= 1) ? kGridCompact : kGridSpeculative;
}

// stage 1: stream generation (LUTs, activation words, weight words + signs) into the workspace.
// allow_partial: a null operand is skipped and what an earlier expand with the same descriptor and workspace wrote
// for it stays in place (a caller whose weights do not change between calls expands them once).
static int conv_expand(const rexsc_sc_conv_desc *desc, const void *d_act, const void *d_weight, void *d_workspace,
                       size_t workspace_bytes, cudaStream_t st, bool allow_partial, int w_seed_pos = 13,
                       int w_seed_neg = 13)
{
    ConvPlan p, pc;
    ConvBuffers b;
    int rc = conv_buffers(desc, d_workspace, workspace_bytes, &p, &b);
    if (rc != REXSC_OK) return rc;
    if (w_seed_pos < 0 || w_seed_neg < 0) return REXSC_E_BAD_ARG;
    p.w_seed_pos = w_seed_pos; // (a local copy of the cached plan; the compact plan below is derived from it)
    p.w_seed_neg = w_seed_neg;
    if (allow_partial ? (!d_act && !d_weight) : (!d_act || !d_weight)) return REXSC_E_BAD_ARG;
    const int k = resolve_kernel(desc, p);
    if (k < 0) return k;
    // The linear generators always use the XOR LFSR (torch_c/sc-extension/sc_cuda_matmul.cu:27-57).
    const int xnor = desc->linear_seeds ? 0 : (desc->xnor ? 1 : 0);
    const int mode = grid_mode(desc, p, k, &pc);
    const ConvPlan &pa = mode == kGridCompact ? pc : p; // the grid the separate activation launches below write
    uint32_t *Ab = static_cast<uint32_t *>(b.tc);
    // the weight planes sit behind the largest (the standard) activation planes, whichever grid is in use
    uint32_t *Wb = reinterpret_cast<uint32_t *>(static_cast<uint8_t *>(b.tc) + conv_tc_weight_offset(p));
    if (k == REXSC_KERNEL_TENSOR && d_act) {
        // one launch for the whole stage (it also clears the status block) where the shape qualifies
        const bool no_w = d_weight == nullptr;
        if (mode == kGridSpeculative) {
            REXSC_CUDA_CHECK(cudaMemsetAsync(b.status, 0, 256, st));
            rc = launch_expand_all_bits(pc, *desc, d_act, d_weight, xnor, Ab, Wb, b.status,
                                        ExpandAllOptions{true, false, no_w}, st);
            if (rc == REXSC_OK) // the standard planes, if the border turned out not to be zero
                rc = launch_expand_all_bits(p, *desc, d_act, d_weight, xnor, Ab, Wb, b.status,
                                            ExpandAllOptions{false, true, true}, st);
        } else {
            rc = launch_expand_all_bits(pa, *desc, d_act, d_weight, xnor, Ab, Wb, b.status,
                                        ExpandAllOptions{false, false, no_w}, st);
        }
        if (rc != REXSC_E_UNSUPPORTED) return rc;
    }
    if (mode == kGridSpeculative) {
        // Separate launches write the standard planes.  Word 1 says so to the accumulate stage; a weights-only call
        // leaves it as the last activation expand set it.
        REXSC_CUDA_CHECK(cudaMemsetAsync(b.status, 0, sizeof(int), st));
        if (d_act) REXSC_CUDA_CHECK(cudaMemsetAsync(reinterpret_cast<char *>(b.status + 1), 1, 1, st));
    } else {
        REXSC_CUDA_CHECK(cudaMemsetAsync(b.status, 0, 256, st));
    }
    rc = launch_build_lut_pair(p.l, desc->bit_length, desc->gen_config, xnor, desc->prog_total_width,
                               desc->prog_load_width, desc->prog_load_wait, b.lut_a, b.lut_w, st);
    if (rc != REXSC_OK) return rc;
    if (k == REXSC_KERNEL_TENSOR) {
        // the tensor-core kernel reads channel-packed bit planes: Ab, then Wb, in the tensor region of the workspace
        if (d_act) {
            rc = launch_expand_act_bits(pa, *desc, d_act, b.lut_a, Ab, st);
            if (rc != REXSC_OK) return rc;
        }
        if (d_weight) rc = launch_expand_weight_bits(p, *desc, d_weight, b.lut_w, Wb, st);
        return rc;
    }
    // the ALU kernels read time-packed stream words
    if (d_act) {
        rc = launch_expand_act(p, *desc, d_act, b.lut_a, b.A, st);
        if (rc != REXSC_OK) return rc;
    }
    if (d_weight) rc = launch_expand_weight(p, *desc, d_weight, b.lut_w, b.Wt, b.S, st);
    return rc;
}

// stage 2: OR-n accumulation over the stream words of the workspace
static int conv_accumulate(const rexsc_sc_conv_desc *desc, int16_t *d_out_pos, int16_t *d_out_neg,
                           void *d_workspace, size_t workspace_bytes, cudaStream_t st)
{
    ConvPlan p, pc;
    ConvBuffers b;
    int rc = conv_buffers(desc, d_workspace, workspace_bytes, &p, &b);
    if (rc != REXSC_OK) return rc;
    if (!d_out_pos || !d_out_neg) return REXSC_E_BAD_ARG;
    const int k = resolve_kernel(desc, p);
    if (k < 0) return k;
    if (k == REXSC_KERNEL_TENSOR) {
        const size_t w_off = conv_tc_weight_offset(p);
        const int mode = grid_mode(desc, p, k, &pc);
        if (mode == kGridStandard) return launch_conv_tc(p, *desc, b.tc, w_off, d_out_pos, d_out_neg, b.status, 0, st);
        if (mode == kGridCompact) return launch_conv_tc(pc, *desc, b.tc, w_off, d_out_pos, d_out_neg, b.status, 0, st);
        // one launch per possible verdict of the expand stage
        rc = launch_conv_tc(pc, *desc, b.tc, w_off, d_out_pos, d_out_neg, b.status, +1, st);
        if (rc != REXSC_OK) return rc;
        return launch_conv_tc(p, *desc, b.tc, w_off, d_out_pos, d_out_neg, b.status, -1, st);
    }
    if (k == REXSC_KERNEL_TILED)
        return launch_conv_tiled(p, *desc, b.A, b.Wt, b.S, d_out_pos, d_out_neg, b.status, st);
    return launch_conv_direct(p, *desc, b.A, b.Wt, b.S, d_out_pos, d_out_neg, st);
}

int conv_forward(const rexsc_sc_conv_desc *desc, const void *d_act, const void *d_weight, int16_t *d_out_pos,
                 int16_t *d_out_neg, void *d_workspace, size_t workspace_bytes, cudaStream_t st, int w_seed_pos,
                 int w_seed_neg)
{
    if (!d_act || !d_weight || !d_out_pos || !d_out_neg) {
        ConvPlan p;
        int rc = make_conv_plan(desc, &p);
        return rc != REXSC_OK ? rc : REXSC_E_BAD_ARG;
    }
    int rc = conv_expand(desc, d_act, d_weight, d_workspace, workspace_bytes, st, false, w_seed_pos, w_seed_neg);
    if (rc != REXSC_OK) return rc;
    return conv_accumulate(desc, d_out_pos, d_out_neg, d_workspace, workspace_bytes, st);
}

static void linear_desc(rexsc_sc_conv_desc *d, int32_t batch, int32_t c_in, int32_t c_out, int32_t act_dtype,
                        int32_t w_dtype, int32_t bit_length, int32_t lfsr_length, int32_t bin_config,
                        int32_t gen_config, int32_t tw, int32_t lw, int32_t lwait)
{
    memset(d, 0, sizeof(*d));
    d->batch = batch; d->c_in = c_in; d->h_in = 1; d->w_in = 1;
    d->c_out = c_out; d->kh = 1; d->kw = 1;
    d->stride_h = 1; d->stride_w = 1;
    d->act_dtype = act_dtype; d->w_dtype = w_dtype;
    // with 1x1 maps and filters NCHW and NHWC are the same memory; channels_last selects the vectorised expansion and
    // lets short grids split their time slots over more CTAs
    d->act_channels_last = 1; d->w_channels_last = 1; d->out_channels_last = 1;
    d->bit_length = bit_length; d->lfsr_length = lfsr_length; d->bin_config = bin_config;
    d->gen_config = gen_config; d->xnor = 0;
    d->prog_total_width = tw; d->prog_load_width = lw; d->prog_load_wait = lwait;
    d->linear_seeds = 1;
    d->kernel = REXSC_KERNEL_AUTO;
}

} // namespace rexsc

using namespace rexsc;

extern "C" int rexsc_abi_version(void) { return REXSC_ABI_VERSION; }

extern "C" const char *rexsc_last_cuda_error(void) { return g_cuda_error; }

extern "C" unsigned long long rexsc_kernel_launch_count(void) { return g_kernel_launches.load(std::memory_order_relaxed); }

extern "C" size_t rexsc_sc_conv2d_workspace_size(const rexsc_sc_conv_desc *desc)
{
    ConvPlan p;
    if (make_conv_plan(desc, &p) != REXSC_OK) return 0;
    return p.total;
}

extern "C" int rexsc_sc_conv2d_kernel_choice(const rexsc_sc_conv_desc *desc)
{
    ConvPlan p;
    int rc = make_conv_plan(desc, &p);
    if (rc != REXSC_OK) return rc;
    if (desc->kernel < REXSC_KERNEL_AUTO || desc->kernel > REXSC_KERNEL_TENSOR) return REXSC_E_BAD_ARG;
    return resolve_kernel(desc, p);
}

extern "C" int rexsc_sc_conv2d_fwd(const rexsc_sc_conv_desc *desc, const void *d_act, const void *d_weight,
                                   int16_t *d_out_pos, int16_t *d_out_neg, void *d_workspace,
                                   size_t workspace_bytes, void *stream)
{
    return conv_forward(desc, d_act, d_weight, d_out_pos, d_out_neg, d_workspace, workspace_bytes,
                        (cudaStream_t)stream);
}

extern "C" int rexsc_sc_conv2d_expand(const rexsc_sc_conv_desc *desc, const void *d_act, const void *d_weight,
                                      void *d_workspace, size_t workspace_bytes, void *stream)
{
    return conv_expand(desc, d_act, d_weight, d_workspace, workspace_bytes, (cudaStream_t)stream, true);
}

extern "C" int rexsc_sc_conv2d_accumulate(const rexsc_sc_conv_desc *desc, int16_t *d_out_pos, int16_t *d_out_neg,
                                          void *d_workspace, size_t workspace_bytes, void *stream)
{
    return conv_accumulate(desc, d_out_pos, d_out_neg, d_workspace, workspace_bytes, (cudaStream_t)stream);
}

extern "C" size_t rexsc_sc_linear_workspace_size(int32_t batch, int32_t c_in, int32_t c_out, int32_t bit_length,
                                                 int32_t lfsr_length, int32_t gen_config)
{
    rexsc_sc_conv_desc d;
    linear_desc(&d, batch, c_in, c_out, REXSC_F32, REXSC_F32, bit_length, lfsr_length, 0, gen_config, 7, 8, 1);
    return rexsc_sc_conv2d_workspace_size(&d);
}

extern "C" int rexsc_sc_linear_fwd(int32_t batch, int32_t c_in, int32_t c_out, int32_t act_dtype, int32_t w_dtype,
                                   int32_t bit_length, int32_t lfsr_length, int32_t bin_config, int32_t gen_config,
                                   int32_t prog_total_width, int32_t prog_load_width, int32_t prog_load_wait,
                                   const void *d_act, const void *d_weight, int16_t *d_out_pos, int16_t *d_out_neg,
                                   void *d_workspace, size_t workspace_bytes, void *stream)
{
    rexsc_sc_conv_desc d;
    linear_desc(&d, batch, c_in, c_out, act_dtype, w_dtype, bit_length, lfsr_length, bin_config, gen_config,
                prog_total_width, prog_load_width, prog_load_wait);
    return conv_forward(&d, d_act, d_weight, d_out_pos, d_out_neg, d_workspace, workspace_bytes,
                        (cudaStream_t)stream);
}

extern "C" int rexsc_sc_linear_fwd_seeded(int32_t batch, int32_t c_in, int32_t c_out, int32_t act_dtype, int32_t w_dtype,
                                          int32_t bit_length, int32_t lfsr_length, int32_t bin_config,
                                          int32_t gen_config, int32_t prog_total_width, int32_t prog_load_width,
                                          int32_t prog_load_wait, int32_t w_seed_pos, int32_t w_seed_neg,
                                          const void *d_act, const void *d_weight, int16_t *d_out_pos,
                                          int16_t *d_out_neg, void *d_workspace, size_t workspace_bytes, void *stream)
{
    rexsc_sc_conv_desc d;
    linear_desc(&d, batch, c_in, c_out, act_dtype, w_dtype, bit_length, lfsr_length, bin_config, gen_config,
                prog_total_width, prog_load_width, prog_load_wait);
    return conv_forward(&d, d_act, d_weight, d_out_pos, d_out_neg, d_workspace, workspace_bytes,
                        (cudaStream_t)stream, w_seed_pos, w_seed_neg);
}

extern "C" int rexsc_workspace_status(const void *d_workspace, void *stream)
{
    if (!d_workspace) return REXSC_E_BAD_ARG;
    int host = 0;
    REXSC_CUDA_CHECK(cudaMemcpyAsync(&host, d_workspace, sizeof(int), cudaMemcpyDeviceToHost, (cudaStream_t)stream));
    REXSC_CUDA_CHECK(cudaStreamSynchronize((cudaStream_t)stream));
    return host == 0 ? REXSC_OK : REXSC_E_DEVICE_TIMEOUT;
}

extern "C" int rexsc_build_lfsr_lut(int32_t lfsr_length, int32_t bit_length, int32_t gen_config, int32_t xnor,
                                    int32_t prog_total_width, int32_t prog_load_width, int32_t prog_load_wait,
                                    int32_t is_weight, uint32_t *d_lut, void *stream)
{
    if (!d_lut) return REXSC_E_BAD_ARG;
    return launch_build_lut(lfsr_length, bit_length, gen_config, xnor ? 1 : 0, prog_total_width, prog_load_width,
                            prog_load_wait, is_weight ? 1 : 0, d_lut, (cudaStream_t)stream);
}

// ---- ALU issue-rate probe ---------------------------------------------------------------------------
__global__ void __launch_bounds__(256) alu_probe_kernel(int iters, uint32_t *sink)
{
    // 16 accumulators, one three-input logic op each, four times per iteration = 64 LOP3 per iteration.
    uint32_t r[16];
    const uint32_t t = blockIdx.x * blockDim.x + threadIdx.x;
#pragma unroll
    for (int i = 0; i < 16; i++) r[i] = t * 2654435761u + i;
    uint32_t a = t ^ 0x9e3779b9u;
    for (int it = 0; it < iters; it++) {
#pragma unroll
        for (int rep = 0; rep < 4; rep++) {
#pragma unroll
            for (int i = 0; i < 16; i++)
                asm volatile("lop3.b32 %0, %0, %1, %2, 0x6a;" : "+r"(r[i]) : "r"(a), "r"(r[(i + 1) & 15]));
        }
        a += 0x01010101u;
    }
    uint32_t x = 0;
#pragma unroll
    for (int i = 0; i < 16; i++) x ^= r[i];
    sink[t] = x;
}

extern "C" int rexsc_alu_probe(int32_t blocks, int32_t iters, uint32_t *d_sink, void *stream)
{
    if (blocks < 1 || iters < 1 || !d_sink) return REXSC_E_BAD_ARG;
    alu_probe_kernel<<<blocks, 256, 0, (cudaStream_t)stream>>>(iters, d_sink);
    REXSC_LAUNCH_CHECK("alu_probe_kernel");
    return REXSC_OK;
}

extern "C" int rexsc_mma_probe(int32_t blocks, int32_t iters, int32_t n_cols, uint32_t *d_sink, void *stream)
{
    return launch_mma_probe(blocks, iters, n_cols, d_sink, (cudaStream_t)stream);
}
