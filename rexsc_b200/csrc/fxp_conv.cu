// FXP fixed-point conv with saturating accumulation.
//
// Reference semantics (torch_c/sc-extension/fixed_cuda_kernel.cu:20-41 adders, :103-120 limits, :153-206
// product order): products are visited in (c_in, kh, kw) order with the dot product zero-padded to a multiple
// of 8, positive and negative weight parts accumulate separately through
//     add(acc, prod) = sat_shift(acc + prod [- (acc*prod) >> 2p for the simulated OR add]),
//     sat_shift(v)   = ((min(v, max) >> d) + ((min(v, max) >> max(0, d-1)) & 1)) << d,
// d = max(0, 2p - p_out), max = ((2^min(31, max(2p, p_out)) - 1) >> d) << d, and the output is pos - neg.
//
// Three kernels (the closed form also has a tensor-core implementation, fxp_conv_umma.cu, used by default):
//   * closed form (add_config 0, d = 0 -- every configuration the reference front end uses): with d = 0 the
//     accumulator is always even after an add, so each add contributes prod + (prod & 1) until the cap:
//         pos = min( sum a*w+ + sum (a&1)(w+&1), 2^pmax ),  all addends >= 0, hence order-free.
//     It is evaluated with packed int8 dot products (dp4a): four products and four parity products per two
//     instructions, and the parity bits ride in a second int8 operand.
//   * sequential (everything else): one thread per output walks the products in the reference's order.
#include "common.cuh"

namespace rexsc {

namespace {

struct FxpArgs {
    int N, C, H, W, Hp, Wp, ph, pw, Co, KH, KW, OH, OW, sh, sw;
    int add_config, p_in, d, max_value;
    long long K, Kp;
    float scale;
};

// round-half-even quantiser of fixed_cuda.cpp:28-30 (torch.round == rintf)
__device__ __forceinline__ int quant_round_unipolar(float x, float scale)
{
    float v = x * scale;
    v = fminf(fmaxf(v, 0.f), scale - 1.f);
    return (int)rintf(v);
}

template <typename T>
__global__ void fxp_quant_act_kernel(FxpArgs a, const T *__restrict__ x, int32_t *__restrict__ q)
{
    long long total = (long long)a.N * a.C * a.Hp * a.Wp;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        int w = (int)(i % a.Wp);
        long long t = i / a.Wp;
        int h = (int)(t % a.Hp);
        long long nc = t / a.Hp;
        int hi = h - a.ph, wi = w - a.pw;
        int v = 0;
        if (hi >= 0 && hi < a.H && wi >= 0 && wi < a.W)
            v = quant_round_unipolar(load_as_float<T>(x, (nc * a.H + hi) * a.W + wi), a.scale);
        q[i] = v;
    }
}

template <typename T>
__global__ void fxp_quant_w_kernel(FxpArgs a, const T *__restrict__ w, int32_t *__restrict__ qp,
                                   int32_t *__restrict__ qn)
{
    long long total = (long long)a.Co * a.K;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        float v = load_as_float<T>(w, i) * a.scale;
        qp[i] = (int)rintf(fminf(fmaxf(v, 0.f), a.scale - 1.f));
        qn[i] = (int)rintf(-fminf(fmaxf(v, 1.f - a.scale), 0.f));
    }
}

__device__ __forceinline__ int sat_shift(int v, int max_value, int d)
{
    int s = min(v, max_value);
    int rb = (s >> max(0, d - 1)) % 2;
    return (int)((unsigned)((s >> d) + rb) << d);
}

struct Or2 { int v1, v2; };
__device__ __forceinline__ Or2 add_or2(Or2 a, Or2 b, int max_value, int p, int d)
{
    long long a1 = a.v1, a2 = a.v2, b1 = b.v1, b2 = b.v2;
    int o1 = a.v1 + b.v1 - (int)((a1 * a2 * b2) >> (p * 4)) - (int)((a2 * b1 * b2) >> (p * 4)) +
             (int)((a1 * a2 * b1 * b2) >> (p * 6));
    int o2 = a.v2 + b.v2 - (int)((a1 * a2 * b1) >> (p * 4)) - (int)((a1 * b1 * b2) >> (p * 4)) +
             (int)((a1 * a2 * b1 * b2) >> (p * 6));
    Or2 r;
    r.v1 = sat_shift(o1, max_value, d);
    r.v2 = sat_shift(o2, max_value, d);
    return r;
}

// one thread per output, products in reference order
__global__ void __launch_bounds__(256) fxp_conv_seq_kernel(FxpArgs a, const int32_t *__restrict__ act,
                                                           const int32_t *__restrict__ wpos,
                                                           const int32_t *__restrict__ wneg,
                                                           int32_t *__restrict__ out)
{
    long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long total = (long long)a.N * a.Co * a.OH * a.OW;
    if (o >= total) return;
    int ow = (int)(o % a.OW);
    long long t = o / a.OW;
    int oh = (int)(t % a.OH);
    t /= a.OH;
    int co = (int)(t % a.Co);
    int n = (int)(t / a.Co);
    const int32_t *abase = act + (((long long)n * a.C) * a.Hp + (long long)oh * a.sh) * a.Wp + (long long)ow * a.sw;
    const int32_t *wp = wpos + (long long)co * a.K;
    const int32_t *wn = wneg + (long long)co * a.K;
    const int p2 = a.p_in * 2;
    int accp = 0, accn = 0;
    Or2 sp = {0, 0}, sn = {0, 0};
    int pend_p = 0, pend_n = 0;
    long long k = 0;
    for (int ci = 0; ci < a.C; ci++)
        for (int kh = 0; kh < a.KH; kh++)
            for (int kw = 0; kw < a.KW; kw++, k++) {
                int av = __ldg(abase + ((long long)ci * a.Hp + kh) * a.Wp + kw);
                int pp = av * __ldg(wp + k), pn = av * __ldg(wn + k);
                if (a.add_config == 0) {
                    accp = sat_shift(accp + pp, a.max_value, a.d);
                    accn = sat_shift(accn + pn, a.max_value, a.d);
                } else if (a.add_config == 1) {
                    accp = sat_shift(accp + pp - ((accp * pp) >> p2), a.max_value, a.d);
                    accn = sat_shift(accn + pn - ((accn * pn) >> p2), a.max_value, a.d);
                } else if ((k & 1) == 0) {
                    pend_p = pp;
                    pend_n = pn;
                } else {
                    Or2 bp = {pend_p, pp}, bn = {pend_n, pn};
                    sp = add_or2(sp, bp, a.max_value, a.p_in, a.d);
                    sn = add_or2(sn, bn, a.max_value, a.p_in, a.d);
                }
            }
    // zero products up to the next multiple of 8 (fixed_cuda_kernel.cu:156-167 pads the tile with zeros)
    for (; k < a.Kp; k++) {
        if (a.add_config < 2) {
            accp = sat_shift(accp, a.max_value, a.d);
            accn = sat_shift(accn, a.max_value, a.d);
        } else if ((k & 1) == 0) {
            pend_p = 0;
            pend_n = 0;
        } else {
            Or2 bp = {pend_p, 0}, bn = {pend_n, 0};
            sp = add_or2(sp, bp, a.max_value, a.p_in, a.d);
            sn = add_or2(sn, bn, a.max_value, a.p_in, a.d);
        }
    }
    out[o] = a.add_config < 2 ? accp - accn : sp.v1 + sp.v2 - sn.v1 - sn.v2;
}

// ---- closed form ----------------------------------------------------------------------------------
// Operands packed for dp4a: four consecutive k (k = (ci*KH + kh)*KW + kw order is irrelevant here, any fixed
// order works because every addend is non-negative) per 32-bit word, values <= 127 fit int8; a second word
// carries the four parity bits.  Weight words are stored k-major so that a warp's output channels read
// consecutive addresses.  One thread computes one output pixel for 8 consecutive output channels.
constexpr int kFxpCo = 8;

__global__ void fxp_pack_w_kernel(FxpArgs a, const int32_t *__restrict__ qp, const int32_t *__restrict__ qn,
                                  int Kw, int Cop, uint32_t *__restrict__ pk)
{
    // pk[((kq*2 + sign)*2 + which)*Cop + co], which: 0 = values, 1 = parity bits
    long long total = (long long)Kw * Cop;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        int co = (int)(i % Cop);
        int kq = (int)(i / Cop);
        uint32_t vp = 0, vn = 0, bp = 0, bn = 0;
        for (int j = 0; j < 4; j++) {
            long long k = (long long)kq * 4 + j;
            int p = 0, n = 0;
            if (co < a.Co && k < a.K) { p = qp[(long long)co * a.K + k]; n = qn[(long long)co * a.K + k]; }
            vp |= (uint32_t)(p & 0xff) << (8 * j);
            vn |= (uint32_t)(n & 0xff) << (8 * j);
            bp |= (uint32_t)(p & 1) << (8 * j);
            bn |= (uint32_t)(n & 1) << (8 * j);
        }
        size_t base = (size_t)kq * 4 * Cop + co;
        pk[base] = vp;
        pk[base + Cop] = bp;
        pk[base + 2 * (size_t)Cop] = vn;
        pk[base + 3 * (size_t)Cop] = bn;
    }
}

__global__ void __launch_bounds__(128) fxp_conv_closed_kernel(FxpArgs a, const int32_t *__restrict__ act,
                                                              const uint32_t *__restrict__ pk, int Kw, int Cop,
                                                              int cap, int32_t *__restrict__ out)
{
    // grid: x = pixel blocks of 128 (over N*OH*OW), y = groups of kFxpCo output channels
    long long m = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    long long M = (long long)a.N * a.OH * a.OW;
    const int co0 = blockIdx.y * kFxpCo;
    if (m >= M) return;
    int ow = (int)(m % a.OW);
    long long t = m / a.OW;
    int oh = (int)(t % a.OH);
    int n = (int)(t / a.OH);
    const int32_t *abase = act + (((long long)n * a.C) * a.Hp + (long long)oh * a.sh) * a.Wp + (long long)ow * a.sw;
    int accp[kFxpCo], accn[kFxpCo];
#pragma unroll
    for (int c = 0; c < kFxpCo; c++) { accp[c] = 0; accn[c] = 0; }
    const int khw = a.KH * a.KW;
    for (int kq = 0; kq < Kw; kq++) {
        uint32_t av = 0, ab = 0;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            long long k = (long long)kq * 4 + j;
            int v = 0;
            if (k < a.K) {
                int ci = (int)(k / khw);
                int r = (int)(k - (long long)ci * khw);
                int kh = r / a.KW, kw = r - kh * a.KW;
                v = __ldg(abase + ((long long)ci * a.Hp + kh) * a.Wp + kw);
            }
            av |= (uint32_t)(v & 0xff) << (8 * j);
            ab |= (uint32_t)(v & 1) << (8 * j);
        }
        const uint32_t *w = pk + (size_t)kq * 4 * Cop + co0;
#pragma unroll
        for (int c = 0; c < kFxpCo; c++) {
            accp[c] = __dp4a((int)av, (int)__ldg(w + c), accp[c]);
            accp[c] = __dp4a((int)ab, (int)__ldg(w + Cop + c), accp[c]);
            accn[c] = __dp4a((int)av, (int)__ldg(w + 2 * (size_t)Cop + c), accn[c]);
            accn[c] = __dp4a((int)ab, (int)__ldg(w + 3 * (size_t)Cop + c), accn[c]);
        }
    }
#pragma unroll
    for (int c = 0; c < kFxpCo; c++) {
        int co = co0 + c;
        if (co < a.Co) {
            size_t oi = (((size_t)n * a.Co + co) * a.OH + oh) * a.OW + ow;
            out[oi] = min(accp[c], cap) - min(accn[c], cap);
        }
    }
}

} // namespace

size_t fxp_umma_workspace_bytes(int N, int C, int Hp, int Wp, int Co, long long K);
bool fxp_umma_supported(int C, int Hp, int Wp, long long K);
int launch_fxp_conv_umma(int N, int C, int H, int W, int ph, int pw, int Co, int KH, int KW, int OH, int OW, int sh,
                         int sw, int cap, float scale, const void *d_act, int act_dtype, const void *d_w, int w_dtype,
                         void *ws, int32_t *out, int *status, bool swizzled, cudaStream_t st);

struct FxpPlan {
    FxpArgs a;
    bool closed, umma;
    int Kw, Cop, cap;
    size_t off_status, off_qa, off_qp, off_qn, off_pk, off_umma, total;
};

static int make_fxp_plan(const rexsc_fxp_conv_desc *d, FxpPlan *p)
{
    if (!d || !p) return REXSC_E_BAD_ARG;
    if (d->batch < 1 || d->c_in < 1 || d->h_in < 1 || d->w_in < 1 || d->c_out < 1 || d->kh < 1 || d->kw < 1)
        return REXSC_E_BAD_ARG;
    if (d->pad_h < 0 || d->pad_w < 0 || d->stride_h < 1 || d->stride_w < 1) return REXSC_E_BAD_ARG;
    if (d->act_dtype < 0 || d->act_dtype > 2 || d->w_dtype < 0 || d->w_dtype > 2) return REXSC_E_BAD_ARG;
    if (d->add_config < 0 || d->precision_in < 1 || d->precision_in > 15 || d->precision_out < 1)
        return REXSC_E_BAD_ARG;
    FxpArgs &a = p->a;
    a.N = d->batch; a.C = d->c_in; a.H = d->h_in; a.W = d->w_in;
    a.ph = d->pad_h; a.pw = d->pad_w; a.sh = d->stride_h; a.sw = d->stride_w;
    a.Hp = a.H + 2 * a.ph; a.Wp = a.W + 2 * a.pw;
    a.Co = d->c_out; a.KH = d->kh; a.KW = d->kw;
    if (a.Hp < a.KH || a.Wp < a.KW) return REXSC_E_BAD_ARG;
    a.OH = (a.Hp - a.KH) / a.sh + 1;
    a.OW = (a.Wp - a.KW) / a.sw + 1;
    a.add_config = d->add_config;
    a.p_in = d->precision_in;
    int pm = d->precision_in * 2 > d->precision_out ? d->precision_in * 2 : d->precision_out;
    if (pm > 31) pm = 31;
    a.d = d->precision_in * 2 - d->precision_out;
    if (a.d < 0) a.d = 0;
    a.max_value = (int)((((unsigned)1 << pm) - 1) >> a.d << a.d);
    a.K = (long long)a.C * a.KH * a.KW;
    a.Kp = (a.K + 7) / 8 * 8;
    a.scale = (float)(1 << d->precision_in);
    long long n_act = (long long)a.N * a.C * a.Hp * a.Wp;
    long long n_out = (long long)a.N * a.Co * a.OH * a.OW;
    if (n_act > 0x7fffffffLL * 2 || n_out > 0x7fffffffLL * 2) return REXSC_E_TOO_LONG;
    // closed form needs: plain add, no shift, int8 operands, no int32 overflow before the cap is applied
    long long worst = a.K * 127LL * 127LL + a.K;
    p->closed = (a.add_config == 0 && a.d == 0 && d->precision_in <= 7 && pm <= 30 && worst < 0x7fffffffLL);
    p->cap = p->closed ? (1 << pm) : 0;
    p->Kw = (int)((a.K + 3) / 4);
    p->Cop = (a.Co + kFxpCo - 1) / kFxpCo * kFxpCo;
    if (d->kernel < 0 || d->kernel > 3) return REXSC_E_BAD_ARG;
    p->umma = p->closed && d->kernel != 1 && fxp_umma_supported(a.C, a.Hp, a.Wp, a.K);
    if (d->kernel >= 2 && !p->umma) return REXSC_E_UNSUPPORTED;
    size_t off = 0;
    p->off_status = off; off += 256;
    // (the tensor-core path quantises straight into its own int8 operands: no int32 intermediates)
    p->off_qa = off; off += p->umma ? 0 : align_up((size_t)n_act * 4, 256);
    p->off_qp = off; off += p->umma ? 0 : align_up((size_t)a.Co * a.K * 4, 256);
    p->off_qn = off; off += p->umma ? 0 : align_up((size_t)a.Co * a.K * 4, 256);
    p->off_pk = off; off += p->umma ? 0 : align_up((size_t)p->Kw * 4 * p->Cop * 4, 256);
    p->off_umma = off;
    if (p->umma) off += fxp_umma_workspace_bytes(a.N, a.C, a.Hp, a.Wp, a.Co, a.K);
    p->total = off;
    return REXSC_OK;
}

} // namespace rexsc

using namespace rexsc;

extern "C" size_t rexsc_fxp_conv2d_workspace_size(const rexsc_fxp_conv_desc *desc)
{
    FxpPlan p;
    if (make_fxp_plan(desc, &p) != REXSC_OK) return 0;
    return p.total;
}

extern "C" int rexsc_fxp_conv2d_fwd(const rexsc_fxp_conv_desc *desc, const void *d_act, const void *d_weight,
                                    int32_t *d_out, void *d_workspace, size_t workspace_bytes, void *stream)
{
    FxpPlan p;
    int rc = make_fxp_plan(desc, &p);
    if (rc != REXSC_OK) return rc;
    if (!d_act || !d_weight || !d_out) return REXSC_E_BAD_ARG;
    if (!d_workspace || workspace_bytes < p.total || (reinterpret_cast<uintptr_t>(d_workspace) & 255))
        return REXSC_E_WORKSPACE;
    cudaStream_t st = (cudaStream_t)stream;
    uint8_t *ws = (uint8_t *)d_workspace;
    int32_t *qa = (int32_t *)(ws + p.off_qa), *qp = (int32_t *)(ws + p.off_qp), *qn = (int32_t *)(ws + p.off_qn);
    uint32_t *pk = (uint32_t *)(ws + p.off_pk);
    int *status = (int *)(ws + p.off_status);
    const FxpArgs &a = p.a;
    REXSC_CUDA_CHECK(cudaMemsetAsync(status, 0, 256, st));
    if (p.umma) // quantises inside its own operand-preparation kernels
        return launch_fxp_conv_umma(a.N, a.C, a.H, a.W, a.ph, a.pw, a.Co, a.KH, a.KW, a.OH, a.OW, a.sh, a.sw, p.cap,
                                    a.scale, d_act, desc->act_dtype, d_weight, desc->w_dtype, ws + p.off_umma, d_out,
                                    status, desc->kernel != 3, st);
    long long n_act = (long long)a.N * a.C * a.Hp * a.Wp;
    unsigned gb = (unsigned)((n_act + 255) / 256 < 148 * 32 ? (n_act + 255) / 256 : 148 * 32);
    switch (desc->act_dtype) {
    case REXSC_F32: fxp_quant_act_kernel<float><<<gb, 256, 0, st>>>(a, (const float *)d_act, qa); break;
    case REXSC_F16: fxp_quant_act_kernel<__half><<<gb, 256, 0, st>>>(a, (const __half *)d_act, qa); break;
    default: fxp_quant_act_kernel<__nv_bfloat16><<<gb, 256, 0, st>>>(a, (const __nv_bfloat16 *)d_act, qa); break;
    }
    REXSC_LAUNCH_CHECK("fxp_quant_act_kernel");
    long long n_w = (long long)a.Co * a.K;
    unsigned wb = (unsigned)((n_w + 255) / 256 < 148 * 32 ? (n_w + 255) / 256 : 148 * 32);
    switch (desc->w_dtype) {
    case REXSC_F32: fxp_quant_w_kernel<float><<<wb, 256, 0, st>>>(a, (const float *)d_weight, qp, qn); break;
    case REXSC_F16: fxp_quant_w_kernel<__half><<<wb, 256, 0, st>>>(a, (const __half *)d_weight, qp, qn); break;
    default: fxp_quant_w_kernel<__nv_bfloat16><<<wb, 256, 0, st>>>(a, (const __nv_bfloat16 *)d_weight, qp, qn); break;
    }
    REXSC_LAUNCH_CHECK("fxp_quant_w_kernel");
    if (p.closed) {
        long long tot = (long long)p.Kw * p.Cop;
        fxp_pack_w_kernel<<<(unsigned)((tot + 255) / 256), 256, 0, st>>>(a, qp, qn, p.Kw, p.Cop, pk);
        REXSC_LAUNCH_CHECK("fxp_pack_w_kernel");
        long long M = (long long)a.N * a.OH * a.OW;
        dim3 grid((unsigned)((M + 127) / 128), (unsigned)(p.Cop / kFxpCo));
        fxp_conv_closed_kernel<<<grid, 128, 0, st>>>(a, qa, pk, p.Kw, p.Cop, p.cap, d_out);
        REXSC_LAUNCH_CHECK("fxp_conv_closed_kernel");
    } else {
        long long n_out = (long long)a.N * a.Co * a.OH * a.OW;
        fxp_conv_seq_kernel<<<(unsigned)((n_out + 255) / 256), 256, 0, st>>>(a, qa, qp, qn, d_out);
        REXSC_LAUNCH_CHECK("fxp_conv_seq_kernel");
    }
    return REXSC_OK;
}
