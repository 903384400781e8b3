// LFSR/comparator bit-stream generation for the SC conv / linear forward.
//
// Design: the stream of an element depends only on (seed index mod (2^l - 1), quantised value), so
// generation is a table lookup.  One small kernel builds the table of time-packed stream words
// (bit t of the word = time slot t); the expand kernels quantise the float tensors and look the words
// up, writing
//   activations: A[word][c][P]            P = stored pixel index over the zero-padded tensor (ConvPlan)
//   weights:     Wt[word][nt][cch][khw][cc][nl]   (one contiguous block per CTA pipeline stage)
//                S[nt][cch][khw][warp]    sign bits: bit (cc*4 + col) set = negative weight
// Only one of the reference's positive / negative weight streams is ever non-zero for a given weight
// (w_pos = ceil(clamp(w*L,0,L-1)), w_neg = ceil(-clamp(w*L,1-L,0)): torch_c/sc-extension/sc_cuda.cpp:92-93),
// and a zero value gives an all-zero stream, so a single word plus a sign bit carries both.
#include <string.h>

#include "common.cuh"

namespace rexsc {

// ---- LFSR step: torch_c/sc-extension/sc_device.cuh:108-248 ----------------------------------
__host__ __device__ __forceinline__ int lfsr_next(int v, int l, int xnor)
{
    int fb;
    switch (l) {
    case 1: return 1 - v;
    case 2: return (v + 1) & 3;
    case 3: fb = ((v >> 2) ^ (v >> 1)) & 1; break;
    case 4: fb = ((v >> 3) ^ (v >> 2)) & 1; break;
    case 5: fb = ((v >> 4) ^ (v >> 2)) & 1; break;
    case 6: fb = ((v >> 5) ^ (v >> 4)) & 1; break;
    case 7: fb = ((v >> 6) ^ (v >> 5)) & 1; break;
    default: fb = ((v >> 7) ^ (v >> 5) ^ (v >> 4) ^ (v >> 3)) & 1; break;
    }
    if (xnor) fb ^= 1;
    return ((v << 1) & ((1 << l) - 1)) | fb;
}

// One thread per (phase, value): run the generator for bit_length steps.
// Generation loop semantics: torch_c/sc-extension/sc_cuda_conv.cu:70-92 (weights), :149-163 (activations):
// advance then compare; progressive-loading mask on the value; int8 storage of state and value; for
// gen_config g the weight bit t lands in slots t*g..t*g+g-1 and the activation bit t in slots
// (t/g)*g*g + j*g + t%g.
struct LutParams {
    int l, bit_length, g, xnor, tw, lw, lwait, words;
};

// stream words of one (seed phase, value) pair into out[0 .. words)
template <typename Store>
__device__ __forceinline__ void lut_entry(const LutParams &lp, int is_weight, int phase, int value, Store store)
{
    int state = (int)(int8_t)(phase + 1 - (lp.xnor ? 1 : 0));
    const int val8 = (int)(int8_t)value;
    uint32_t acc[32]; // words <= 32 (slots <= 1024)
#pragma unroll 1
    for (int j = 0; j < lp.words; j++) acc[j] = 0u;
#pragma unroll 1
    for (int t = 0; t < lp.bit_length; t++) {
        int cur = (t / lp.lwait + 1) * lp.lw - 1;
        if (cur > lp.tw) cur = lp.tw;
        const int sh = lp.tw - cur;
        const int actual = (val8 >> sh) << sh;
        state = (int)(int8_t)lfsr_next(state, lp.l, lp.xnor);
        if (actual > state) {
            for (int j = 0; j < lp.g; j++) {
                const int slot = is_weight ? t * lp.g + j : (t / lp.g) * lp.g * lp.g + j * lp.g + t % lp.g;
                acc[slot >> 5] |= 1u << (slot & 31);
            }
        }
    }
    for (int j = 0; j < lp.words; j++) store(j, acc[j]);
}

// blockIdx.y = 0: the table `lut` for generator kind `is_weight`; blockIdx.y = 1 (pair launch): the weight table lut_w
__global__ void build_lut_kernel(LutParams lp, int is_weight, uint32_t *__restrict__ lut, uint32_t *__restrict__ lut_w)
{
    if (blockIdx.y == 1) { is_weight = 1; lut = lut_w; }
    const int nvals = 1 << lp.l;
    const int period = nvals - 1;
    const int idx = blockIdx.x * blockDim.x + threadIdx.x;
    if (idx >= period * nvals) return;
    const int phase = idx / nvals;
    const int value = idx - phase * nvals;
    lut_entry(lp, is_weight, phase, value, [&](int j, uint32_t v) { lut[(size_t)idx * lp.words + j] = v; });
}

int launch_build_lut(int l, int bit_length, int gen_config, int xnor, int tw, int lw, int lwait, int is_weight,
                     uint32_t *d_lut, cudaStream_t st)
{
    if (l < 1 || l > 8 || bit_length < 1 || gen_config < 1 || lwait < 1) return REXSC_E_BAD_ARG;
    int slots = bit_length * gen_config;
    if (slots > 1024) return REXSC_E_TOO_LONG;
    int words = (slots + 31) / 32;
    int total = ((1 << l) - 1) * (1 << l);
    LutParams lp{l, bit_length, gen_config, xnor, tw, lw, lwait, words};
    build_lut_kernel<<<(total + 127) / 128, 128, 0, st>>>(lp, is_weight, d_lut, nullptr);
    REXSC_LAUNCH_CHECK("build_lut_kernel");
    return REXSC_OK;
}

// activation and weight tables of one conv call in a single launch
int launch_build_lut_pair(int l, int bit_length, int gen_config, int xnor, int tw, int lw, int lwait, uint32_t *d_lut_a,
                          uint32_t *d_lut_w, cudaStream_t st)
{
    if (l < 1 || l > 8 || bit_length < 1 || gen_config < 1 || lwait < 1) return REXSC_E_BAD_ARG;
    const int slots = bit_length * gen_config;
    if (slots > 1024) return REXSC_E_TOO_LONG;
    const int words = (slots + 31) / 32;
    const int total = ((1 << l) - 1) * (1 << l);
    LutParams lp{l, bit_length, gen_config, xnor, tw, lw, lwait, words};
    build_lut_kernel<<<dim3((total + 127) / 128, 2), 128, 0, st>>>(lp, 0, d_lut_a, d_lut_w);
    REXSC_LAUNCH_CHECK("build_lut_kernel");
    return REXSC_OK;
}

// ---- plan ---------------------------------------------------------------------------------
static int lfsr_length_for(int bit_length)
{
    // torch_c/sc-extension/sc_cuda_kernel.cu:594-619 (2 and 4 fall through to 3)
    switch (bit_length) {
    case 2: case 4: case 8: return 3;
    case 16: return 4;
    case 32: return 5;
    case 64: return 6;
    case 128: return 7;
    case 256: return 8;
    default: return -1;
    }
}

static int make_conv_plan_uncached(const rexsc_sc_conv_desc *d, ConvPlan *p);

// Plans are pure functions of the descriptor; a call derives its plan several times (size query, expand,
// accumulate) and a network repeats a handful of descriptors, so the last few are kept per host thread.
int make_conv_plan(const rexsc_sc_conv_desc *d, ConvPlan *p)
{
    if (!d || !p) return REXSC_E_BAD_ARG;
    struct Entry { rexsc_sc_conv_desc key; ConvPlan plan; bool used; };
    constexpr int kEntries = 64;
    static thread_local Entry cache[kEntries];
    static thread_local int next = 0;
    rexsc_sc_conv_desc key = *d;
    key.kernel = 0; // the kernel choice does not enter the plan
    for (int i = 0; i < kEntries; i++)
        if (cache[i].used && memcmp(&cache[i].key, &key, sizeof(key)) == 0) {
            *p = cache[i].plan;
            return REXSC_OK;
        }
    int rc = make_conv_plan_uncached(d, p);
    if (rc != REXSC_OK) return rc;
    Entry &e = cache[next];
    next = (next + 1) % kEntries;
    e.key = key;
    e.plan = *p;
    e.used = true;
    return REXSC_OK;
}

static int make_conv_plan_uncached(const rexsc_sc_conv_desc *d, ConvPlan *p)
{
    if (!d || !p) return REXSC_E_BAD_ARG;
    if (d->batch < 1 || d->c_in < 1 || d->h_in < 1 || d->w_in < 1 || d->c_out < 1 || d->kh < 1 || d->kw < 1)
        return REXSC_E_BAD_ARG;
    if (d->pad_h < 0 || d->pad_w < 0 || d->stride_h < 1 || d->stride_w < 1) return REXSC_E_BAD_ARG;
    if (d->act_dtype < 0 || d->act_dtype > 2 || d->w_dtype < 0 || d->w_dtype > 2) return REXSC_E_BAD_ARG;
    if (d->bit_length < 1 || d->gen_config < 1 || d->prog_load_wait < 1) return REXSC_E_BAD_ARG;
    if (d->bin_config < 0) return REXSC_E_UNSUPPORTED; // "exactly n" variants are not on the reference GEMM path
    int l = d->lfsr_length > 0 ? d->lfsr_length : lfsr_length_for(d->bit_length);
    // l = 8 is left out: the reference keeps LFSR state and value in int8 storage
    // (torch_c/sc-extension/sc_cuda_conv.cu:37-40), which wraps negative for 8-bit values and makes a
    // zero weight produce a non-zero stream; no reference configuration uses it.
    if (l < 1 || l > 7) return REXSC_E_UNSUPPORTED;
    p->l = l;
    p->nvals = 1 << l;
    p->scale = d->lfsr_length > 0 ? (1 << l) : d->bit_length;
    if (p->scale > p->nvals) return REXSC_E_UNSUPPORTED;
    p->period = p->nvals - 1;
    p->slots = d->bit_length * d->gen_config;
    if (p->slots > 1024) return REXSC_E_TOO_LONG;
    p->words = (p->slots + 31) / 32;
    p->n_or = d->bin_config + 1;
    p->N = d->batch; p->C = d->c_in; p->H = d->h_in; p->W = d->w_in;
    p->ph = d->pad_h; p->pw = d->pad_w; p->sh = d->stride_h; p->sw = d->stride_w;
    p->Hp = d->h_in + 2 * d->pad_h;
    p->Wp = d->w_in + 2 * d->pad_w;
    p->Co = d->c_out; p->KH = d->kh; p->KW = d->kw; p->KHW = d->kh * d->kw;
    if (p->Hp < p->KH || p->Wp < p->KW) return REXSC_E_BAD_ARG;
    p->OH = (p->Hp - p->KH) / p->sh + 1;
    p->OW = (p->Wp - p->KW) / p->sw + 1;
    p->nrh = p->sh < p->KH ? p->sh : p->KH;
    p->nrw = p->sw < p->KW ? p->sw : p->KW;
    p->Wq = (p->Wp + p->sw - 1) / p->sw;
    p->Hrows = (p->Hp + p->sh - 1) / p->sh * p->nrh;
    p->Wrow = p->Wq * p->nrw;
    p->M = (long long)p->N * p->OH * p->OW;
    {
        // Row pitch: the 32 lanes of a warp read the words of 32 consecutive output pixels; when a warp spans
        // several output rows (narrow feature maps) the pitch decides how many of those words share a
        // shared-memory bank.  Pick the padding (< 32 words) with the fewest bank passes per load, weighing
        // passes against the memory the padding costs.
        const int base = p->Wrow;
        double best_cost = 1e30;
        int best_pitch = base;
        auto max_tap_for = [&](int pitch) {
            int mt = 0;
            for (int kh = 0; kh < p->KH; kh++)
                for (int kw = 0; kw < p->KW; kw++) {
                    int t = tap_offset(kh, kw, p->sh, p->sw, p->nrh, pitch, p->Wq);
                    if (t > mt) mt = t;
                }
            return mt;
        };
        // largest tile (256, else 128 pixels) whose patch fits the tiled kernel's stage at the unpadded pitch;
        // padding must not push that tile out of the stage
        int fit_bm = 0;
        for (int bm = 256; bm >= 128 && !fit_bm; bm -= 128)
            if (patch_bound_words(bm, p->M, p->OW, p->OH, p->nrh, p->Hrows, base, max_tap_for(base)) <= kPlaneWords)
                fit_bm = bm;
        for (int pad = 0; pad < 32; pad++) {
            const int pitch = base + pad;
            if (pad > 0 && fit_bm &&
                patch_bound_words(fit_bm, p->M, p->OW, p->OH, p->nrh, p->Hrows, pitch, max_tap_for(pitch)) > kPlaneWords)
                continue;
            const long long img = (long long)p->Hrows * pitch;
            double passes = 0;
            int samples = 0;
            for (long long m0 = 0; m0 < p->M && samples < 64; m0 += 32, samples++) {
                int cnt[32] = {0};
                int worst = 0;
                for (int lane = 0; lane < 32 && m0 + lane < p->M; lane++) {
                    const long long m = m0 + lane;
                    const long long ow = m % p->OW, t = m / p->OW, oh = t % p->OH, n = t / p->OH;
                    const int bank = (int)((n * img + oh * (long long)p->nrh * pitch + ow) & 31);
                    if (++cnt[bank] > worst) worst = cnt[bank];
                }
                passes += worst;
            }
            const double cost = passes / samples * (1.0 + 1.0 * pad / base);
            if (cost < best_cost - 1e-9) { best_cost = cost; best_pitch = pitch; }
        }
        p->Wrow = best_pitch;
    }
    p->max_tap = 0;
    for (int kh = 0; kh < p->KH; kh++)
        for (int kw = 0; kw < p->KW; kw++) {
            int t = tap_offset(kh, kw, p->sh, p->sw, p->nrh, p->Wrow, p->Wq);
            if (t > p->max_tap) p->max_tap = t;
        }
    p->NHW = (long long)p->N * p->Hrows * p->Wrow;
    p->NHWp = (p->NHW + 3) / 4 * 4;
    p->Cpad = (p->C + kChunkC - 1) / kChunkC * kChunkC;
    p->CCH = p->Cpad / kChunkC;
    p->NT = (p->Co + kTileN - 1) / kTileN;
    p->Kdot = (long long)p->C * p->KHW;
    // the per-slot counters of the generic path are 16 bits wide, like the reference's (sc_device.cuh:380-384)
    if (p->Kdot > 65535) return REXSC_E_TOO_LONG;
    if (p->NHWp > 0x7fffffffLL || p->M > 0x7fffffffLL) return REXSC_E_TOO_LONG;
    p->a_plane_words = (long long)p->Cpad * p->NHWp;
    p->w_plane_words = (long long)p->NT * p->CCH * p->KHW * kChunkC * kTileN;
    size_t lut_bytes = (size_t)p->period * p->nvals * p->words * sizeof(uint32_t);
    size_t off = 0;
    p->off_status = off; off += 256;
    p->off_lut_a = off; off += align_up(lut_bytes, 256);
    p->off_lut_w = off; off += align_up(lut_bytes, 256);
    p->off_A = off; off += align_up((size_t)p->words * p->a_plane_words * sizeof(uint32_t), 256);
    p->off_Wt = off; off += align_up((size_t)p->words * p->w_plane_words * sizeof(uint32_t), 256);
    p->off_S = off; off += align_up((size_t)p->NT * p->CCH * p->KHW * (kTileN / kWarpN) * sizeof(uint32_t), 256);
    p->off_tc = off;
    p->tc_ok = conv_tc_supported(*p);
    if (p->tc_ok) off += conv_tc_workspace_bytes(*p);
    p->total = off;
    return REXSC_OK;
}

// ---- activation expansion -------------------------------------------------------------------
// Seed index of an activation element: c*Hp*Wp + h*Wp + w on the PADDED tensor, offset 0
// (torch_c/sc-extension/sc_cuda_conv.cu:133,139); linear: c only (sc_cuda_matmul.cu:177).
struct ExpandActArgs {
    int N, C, H, W, Hp, Wp, ph, pw, Cpad;
    int sh, sw, nrh, nrw, Wq, Hrows, Wrow;
    uint32_t plane_mod; // (Hp * Wp) mod period
    long long NHW, NHWp, a_plane_words;
    int period, nvals, words, linear_seeds;
    float scale;
};

// stored pixel index -> (n, h, w) of the padded tensor; false for slots that hold no pixel (they stay zero)
__device__ __forceinline__ bool decode_pixel(const ExpandActArgs &a, long long P64, int &n, int &h, int &w)
{
    const uint32_t P = (uint32_t)P64; // stored pixel indices fit 31 bits (checked when the plan is made)
    const int col = (int)(P % (uint32_t)a.Wrow);
    const uint32_t t = P / (uint32_t)a.Wrow;
    const int row = (int)(t % (uint32_t)a.Hrows);
    n = (int)(t / (uint32_t)a.Hrows);
    h = (row / a.nrh) * a.sh + row % a.nrh;
    w = (col % a.Wq) * a.sw + col / a.Wq;
    return col < a.Wq * a.nrw && h < a.Hp && w < a.Wp; // pitch padding holds no pixel
}

// One CTA expands a tile of 32 stored pixels x 32 channels.  NHWC inputs are read with the channel index
// fastest (one 128-byte row per pixel and warp), quantised, transposed through shared memory and written with
// the pixel index fastest (one 128-byte run per channel and warp); NCHW inputs need no transpose.
template <typename T, bool NHWC>
__global__ void __launch_bounds__(256) expand_act_kernel(ExpandActArgs a, const T *__restrict__ x,
                                                         const uint32_t *__restrict__ lut, uint32_t *__restrict__ A)
{
    __shared__ uint8_t q_s[32][36]; // [channel][pixel], padded
    const int tx = threadIdx.x & 31, ty = threadIdx.x >> 5;
    const long long P0 = (long long)blockIdx.x * 32;
    const int c0 = blockIdx.y * 32;
    if (NHWC) {
        const int c = c0 + tx;
#pragma unroll
        for (int i = 0; i < 4; i++) {
            const int pl = ty + 8 * i;
            const long long P = P0 + pl;
            int q = 0;
            int n, h, w;
            if (P < a.NHW && c < a.C && decode_pixel(a, P, n, h, w)) {
                const int hi = h - a.ph, wi = w - a.pw;
                if (hi >= 0 && hi < a.H && wi >= 0 && wi < a.W) {
                    const long long xi = (((long long)n * a.H + hi) * a.W + wi) * a.C + c;
                    q = quant_ceil_unipolar(load_as_float<T>(x, xi), a.scale);
                }
            }
            q_s[tx][pl] = (uint8_t)q;
        }
        __syncthreads();
    }
    const long long P = P0 + tx;
    if (P >= a.NHWp) return;
    int n = 0, h = 0, w = 0;
    const bool pixel_live = P < a.NHW && decode_pixel(a, P, n, h, w);
    const int hi = h - a.ph, wi = w - a.pw;
    const bool inside = pixel_live && hi >= 0 && hi < a.H && wi >= 0 && wi < a.W;
    // seed index c*Hp*Wp + h*Wp + w reduced modulo the LFSR period with 32-bit arithmetic
    const uint32_t hw_mod = ((uint32_t)h * (uint32_t)a.Wp + (uint32_t)w) % (uint32_t)a.period;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int c = c0 + ty + 8 * i;
        if (c >= a.Cpad) break;
        int q = 0;
        if (inside && c < a.C) {
            if (NHWC) {
                q = q_s[ty + 8 * i][tx];
            } else {
                const long long xi = (((long long)n * a.C + c) * a.H + hi) * a.W + wi;
                q = quant_ceil_unipolar(load_as_float<T>(x, xi), a.scale);
            }
        }
        const uint32_t phase = a.linear_seeds ? (uint32_t)c % (uint32_t)a.period
                                              : ((uint32_t)c * a.plane_mod + hw_mod) % (uint32_t)a.period;
        const uint32_t *row = lut + ((size_t)phase * a.nvals + q) * a.words;
        for (int j = 0; j < a.words; j++) {
            const uint32_t v = q > 0 ? __ldg(row + j) : 0u;
            A[(size_t)j * a.a_plane_words + (size_t)c * a.NHWp + P] = v;
        }
    }
}

template <typename T>
static int expand_act_dispatch(const ExpandActArgs &a, bool nhwc, const void *x, const uint32_t *lut, uint32_t *A,
                               cudaStream_t st)
{
    dim3 grid((unsigned)((a.NHWp + 31) / 32), (unsigned)((a.Cpad + 31) / 32));
    if (grid.y > 65535) return REXSC_E_TOO_LONG;
    if (nhwc)
        expand_act_kernel<T, true><<<grid, 256, 0, st>>>(a, (const T *)x, lut, A);
    else
        expand_act_kernel<T, false><<<grid, 256, 0, st>>>(a, (const T *)x, lut, A);
    REXSC_LAUNCH_CHECK("expand_act_kernel");
    return REXSC_OK;
}

int launch_expand_act(const ConvPlan &p, const rexsc_sc_conv_desc &d, const void *d_act, const uint32_t *d_lut,
                      uint32_t *d_A, cudaStream_t st)
{
    ExpandActArgs a;
    a.N = p.N; a.C = p.C; a.H = p.H; a.W = p.W; a.Hp = p.Hp; a.Wp = p.Wp; a.ph = p.ph; a.pw = p.pw;
    a.Cpad = p.Cpad; a.NHW = p.NHW; a.NHWp = p.NHWp; a.a_plane_words = p.a_plane_words;
    a.sh = p.sh; a.sw = p.sw; a.nrh = p.nrh; a.nrw = p.nrw; a.Wq = p.Wq; a.Hrows = p.Hrows; a.Wrow = p.Wrow;
    a.plane_mod = (uint32_t)(((long long)p.Hp * p.Wp) % p.period);
    a.period = p.period; a.nvals = p.nvals; a.words = p.words; a.linear_seeds = d.linear_seeds;
    a.scale = (float)p.scale;
    bool nhwc = d.act_channels_last != 0;
    switch (d.act_dtype) {
    case REXSC_F32: return expand_act_dispatch<float>(a, nhwc, d_act, d_lut, d_A, st);
    case REXSC_F16: return expand_act_dispatch<__half>(a, nhwc, d_act, d_lut, d_A, st);
    case REXSC_BF16: return expand_act_dispatch<__nv_bfloat16>(a, nhwc, d_act, d_lut, d_A, st);
    }
    return REXSC_E_BAD_ARG;
}

// ---- activation expansion straight to bit planes (operand format of the tensor-core kernel) ---------------------
// Ab[slot][cw][P], bit b = channel 32*cw + b.  One warp owns 32 stored pixels x 32 channels: it quantises them into a
// private byte tile reading along the input's fastest dimension, then every lane takes ONE pixel: it looks up the
// stream words of that pixel's 32 channels (bit t = slot t), transposes the 32 x 32 bit matrix in its registers, and
// holds the 32 slot words (bit b = channel b) -- so each slot's store is one 128-byte run over the warp's pixels.
// The time-packed stream words never touch memory.
__device__ __forceinline__ void transpose32_regs(uint32_t (&v)[32])
{
    // block swap at distances 16, 8, 4, 2, 1: element (row k, column c + j) <-> (row k + j, column c)
#pragma unroll
    for (int j = 16; j >= 1; j >>= 1) {
        const uint32_t m = j == 16 ? 0x0000ffffu : j == 8 ? 0x00ff00ffu : j == 4 ? 0x0f0f0f0fu : j == 2 ? 0x33333333u : 0x55555555u;
#pragma unroll
        for (int k = 0; k < 32; k++) {
            if ((k & j) == 0) {
                const uint32_t t = ((v[k] >> j) ^ v[k + j]) & m;
                v[k + j] ^= t;
                v[k] ^= t << j;
            }
        }
    }
}

// SMEM_LUT: the stream table (a few KB at the common stream lengths) is copied into shared memory first.  A warp's 32
// lookups are a random gather; from L1 that costs one tag pass per distinct 128-byte line (about 20 per load for a
// 4 KB table), from shared memory one pass per bank conflict (about 3).  Each warp then works through kItemsPerWarp
// items so that the copy is amortised.
constexpr int kActItemsPerWarp = 4;
template <typename T, bool NHWC, bool SMEM_LUT>
__global__ void __launch_bounds__(256, 3) expand_act_bits_kernel(ExpandActArgs a, const T *__restrict__ x,
                                                              const uint32_t *__restrict__ lut_g, uint32_t *__restrict__ Ab,
                                                              int CW, long long items)
{
    __shared__ uint8_t q_s[8][32][36];   // [warp][pixel][channel], padded: a lane's row starts in its own bank
    __shared__ long long xb_s[8][32];    // [warp][pixel] input offset of the pixel's channel 0
    extern __shared__ __align__(16) uint32_t lut_s[];
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (SMEM_LUT) {
        const int lut_words = a.period * a.nvals * a.words;
        for (int i = threadIdx.x; i < lut_words; i += blockDim.x) lut_s[i] = __ldg(lut_g + i);
        __syncthreads();
    }
    const uint32_t *lut = SMEM_LUT ? lut_s : lut_g;
    const int n_iter = SMEM_LUT ? kActItemsPerWarp : 1;
    for (int it = 0; it < n_iter; it++) {
    // neighbouring warps: the channel words of the same pixels
    const long long item = ((long long)blockIdx.x * n_iter + it) * 8 + warp;
    if (item >= items) return; // warp-uniform, and no block-wide barrier follows
    const int cw = (int)(item % CW);
    const long long P0 = (item / CW) * 32;
    const int c0 = cw * 32;
    // lane = pixel: where it sits in the input
    int n = 0, h = 0, w = 0;
    const long long P = P0 + lane;
    const bool live = P < a.NHW && decode_pixel(a, P, n, h, w);
    const int hi = h - a.ph, wi = w - a.pw;
    const bool inside = live && hi >= 0 && hi < a.H && wi >= 0 && wi < a.W;
    const uint32_t hw_mod = ((uint32_t)h * (uint32_t)a.Wp + (uint32_t)w) % (uint32_t)a.period;
    const long long xbase = NHWC ? (((long long)n * a.H + hi) * a.W + wi) * a.C : (((long long)n * a.C) * a.H + hi) * a.W + wi;
    // quantise the 32 x 32 tile, reading along the input's fastest dimension
    // (the loads of a batch are all issued before the first value is used: the kernel lives on memory-level
    // parallelism, its occupancy is limited by the 32 live words of the transpose)
    constexpr int kBatch = 16;
    if (NHWC) {
        // lane = channel; the pixels' base offsets are handed over through shared memory (-1: padding, no load)
        xb_s[warp][lane] = inside ? xbase : -1;
        __syncwarp();
        const int c = c0 + lane;
#pragma unroll
        for (int p0 = 0; p0 < 32; p0 += kBatch) {
            float val[kBatch];
#pragma unroll
            for (int i = 0; i < kBatch; i++) {
                const long long xb = xb_s[warp][p0 + i];
                val[i] = (xb >= 0 && c < a.C) ? load_as_float<T>(x, xb + c) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < kBatch; i++) q_s[warp][p0 + i][lane] = (uint8_t)quant_ceil_unipolar(val[i], a.scale);
        }
    } else {
        const long long plane = (long long)a.H * a.W;
#pragma unroll
        for (int cc0 = 0; cc0 < 32; cc0 += kBatch) {
            float val[kBatch];
#pragma unroll
            for (int i = 0; i < kBatch; i++) {
                const int c = c0 + cc0 + i;
                val[i] = (inside && c < a.C) ? load_as_float<T>(x, xbase + c * plane) : 0.f;
            }
#pragma unroll
            for (int i = 0; i < kBatch; i++) q_s[warp][lane][cc0 + i] = (uint8_t)quant_ceil_unipolar(val[i], a.scale);
        }
    }
    __syncwarp();
    // lane = pixel; the channel part of the seed phase is the same for all lanes and advances by a constant
    const uint32_t period = (uint32_t)a.period;
    const uint32_t step_mod = a.linear_seeds ? 1u % period : a.plane_mod % period;
    const uint32_t phase0 = a.linear_seeds ? (uint32_t)c0 % period : (uint32_t)(((unsigned long long)c0 * a.plane_mod) % period);
    const uint32_t pix_mod = a.linear_seeds ? 0u : hw_mod;
    const bool store_ok = P0 + lane < a.NHWp;
    for (int wd = 0; wd < a.words; wd++) {
        uint32_t v[32];
        uint32_t cph = phase0;
#pragma unroll
        for (int cc = 0; cc < 32; cc++) {
            const int q = q_s[warp][lane][cc];
            uint32_t phase = cph + pix_mod;
            if (phase >= period) phase -= period;
            v[cc] = q > 0 ? (SMEM_LUT ? lut[(phase * (uint32_t)a.nvals + (uint32_t)q) * (uint32_t)a.words + (uint32_t)wd]
                                      : __ldg(lut + ((size_t)phase * a.nvals + q) * a.words + wd)) : 0u;
            cph += step_mod;
            if (cph >= period) cph -= period;
        }
        transpose32_regs(v);
        if (store_ok) {
            uint32_t *dst = Ab + ((size_t)(wd * 32) * CW + cw) * a.NHWp + P0 + lane;
            const size_t slot_stride = (size_t)CW * a.NHWp;
#pragma unroll
            for (int t = 0; t < 32; t++) {
                *dst = v[t];
                dst += slot_stride;
            }
        }
    }
    __syncwarp(); // the warp's tiles are rewritten by its next item
    }
}

int launch_expand_act_bits(const ConvPlan &p, const rexsc_sc_conv_desc &d, const void *d_act, const uint32_t *d_lut,
                           uint32_t *d_Ab, cudaStream_t st)
{
    ExpandActArgs a;
    a.N = p.N; a.C = p.C; a.H = p.H; a.W = p.W; a.Hp = p.Hp; a.Wp = p.Wp; a.ph = p.ph; a.pw = p.pw;
    a.Cpad = p.Cpad; a.NHW = p.NHW; a.NHWp = p.NHWp; a.a_plane_words = p.a_plane_words;
    a.sh = p.sh; a.sw = p.sw; a.nrh = p.nrh; a.nrw = p.nrw; a.Wq = p.Wq; a.Hrows = p.Hrows; a.Wrow = p.Wrow;
    a.plane_mod = (uint32_t)(((long long)p.Hp * p.Wp) % p.period);
    a.period = p.period; a.nvals = p.nvals; a.words = p.words; a.linear_seeds = d.linear_seeds;
    a.scale = (float)p.scale;
    const int CW = (p.C + 31) / 32;
    const long long items = ((p.NHWp + 31) / 32) * CW;
    const size_t lut_bytes = (size_t)p.period * p.nvals * p.words * sizeof(uint32_t);
    const bool smem_lut = lut_bytes <= 16 * 1024; // larger tables (stream lengths above 64) stay in global memory / L1
    const int per_warp = smem_lut ? kActItemsPerWarp : 1;
    const long long blocks = (items + 8 * per_warp - 1) / (8 * per_warp);
    if (blocks > 0x7fffffffLL) return REXSC_E_TOO_LONG;
    const bool nhwc = d.act_channels_last != 0;
#define REXSC_ACT_BITS2(T, NHWC_, SM_)                                                                                  \
    expand_act_bits_kernel<T, NHWC_, SM_><<<(unsigned)blocks, 256, SM_ ? lut_bytes : 0, st>>>((a), (const T *)d_act, d_lut, d_Ab, CW, items)
#define REXSC_ACT_BITS(T)                                                                                              \
    do {                                                                                                               \
        if (nhwc) { if (smem_lut) REXSC_ACT_BITS2(T, true, true); else REXSC_ACT_BITS2(T, true, false); }              \
        else { if (smem_lut) REXSC_ACT_BITS2(T, false, true); else REXSC_ACT_BITS2(T, false, false); }                 \
    } while (0)
    switch (d.act_dtype) {
    case REXSC_F32: REXSC_ACT_BITS(float); break;
    case REXSC_F16: REXSC_ACT_BITS(__half); break;
    case REXSC_BF16: REXSC_ACT_BITS(__nv_bfloat16); break;
    default: return REXSC_E_BAD_ARG;
    }
#undef REXSC_ACT_BITS
#undef REXSC_ACT_BITS2
    REXSC_LAUNCH_CHECK("expand_act_bits_kernel");
    return REXSC_OK;
}

// ---- weight expansion -----------------------------------------------------------------------
// Seed index of a weight element: c*KH*KW + kh*KW + kw, offset 13 for both signs
// (torch_c/sc-extension/sc_cuda_conv.cu:45,55-56; sc_device.cuh:33-34); linear: c only.
struct ExpandWArgs {
    int C, Co, KH, KW, KHW, CCH, NT;
    int period, nvals, words, linear_seeds, ohwi;
    long long w_plane_words;
    float scale;
};

template <typename T>
__global__ void __launch_bounds__(256) expand_weight_kernel(ExpandWArgs a, const T *__restrict__ wt,
                                                            const uint32_t *__restrict__ lut,
                                                            uint32_t *__restrict__ Wt, uint32_t *__restrict__ S)
{
    // one warp per (nt, cch, khw, warp8); lane = cc*4 + col
    long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    long long total_warps = (long long)a.NT * a.CCH * a.KHW * 8;
    if (gw >= total_warps) return;
    int w8 = (int)(gw & 7);
    long long t = gw >> 3;
    int khw = (int)(t % a.KHW);
    t /= a.KHW;
    int cch = (int)(t % a.CCH);
    int nt = (int)(t / a.CCH);
    int cc = lane >> 2, col = lane & 3;
    int ci = cch * kChunkC + cc;
    int nl = w8 * kWarpN + col;
    int co = nt * kTileN + nl;
    int kh = khw / a.KW, kw = khw - kh * a.KW;
    int mag = 0;
    bool neg = false;
    if (ci < a.C && co < a.Co) {
        long long wi = a.ohwi ? (((long long)co * a.KH + kh) * a.KW + kw) * a.C + ci
                              : (((long long)co * a.C + ci) * a.KH + kh) * a.KW + kw;
        float v = load_as_float<T>(wt, wi) * a.scale;
        // w_pos = ceil(clamp(v, 0, L-1)); w_neg = ceil(-clamp(v, 1-L, 0))  (sc_cuda.cpp:92-93)
        int qp = (int)ceilf(fminf(fmaxf(v, 0.f), a.scale - 1.f));
        int qn = (int)ceilf(-fminf(fmaxf(v, 1.f - a.scale), 0.f));
        if (qn > 0) { neg = true; mag = qn; } else { mag = qp; }
    }
    long long seed_ind = a.linear_seeds ? (long long)ci : ((long long)ci * a.KH + kh) * a.KW + kw;
    int phase = (int)((13 + seed_ind) % a.period);
    const uint32_t *row = lut + ((size_t)phase * a.nvals + mag) * a.words;
    size_t base = ((((size_t)nt * a.CCH + cch) * a.KHW + khw) * kChunkC + cc) * kTileN + nl;
    for (int j = 0; j < a.words; j++) {
        uint32_t v = mag > 0 ? __ldg(row + j) : 0u;
        Wt[(size_t)j * a.w_plane_words + base] = v;
    }
    unsigned mask = __ballot_sync(0xffffffffu, neg);
    if (lane == 0) S[gw] = mask;
}

int launch_expand_weight(const ConvPlan &p, const rexsc_sc_conv_desc &d, const void *d_w, const uint32_t *d_lut,
                         uint32_t *d_Wt, uint32_t *d_S, cudaStream_t st)
{
    ExpandWArgs a;
    a.C = p.C; a.Co = p.Co; a.KH = p.KH; a.KW = p.KW; a.KHW = p.KHW; a.CCH = p.CCH; a.NT = p.NT;
    a.period = p.period; a.nvals = p.nvals; a.words = p.words; a.linear_seeds = d.linear_seeds;
    a.ohwi = d.w_channels_last; a.w_plane_words = p.w_plane_words; a.scale = (float)p.scale;
    long long total_threads = (long long)p.NT * p.CCH * p.KHW * 8 * 32;
    unsigned blocks = (unsigned)((total_threads + 255) / 256);
    switch (d.w_dtype) {
    case REXSC_F32:
        expand_weight_kernel<float><<<blocks, 256, 0, st>>>(a, (const float *)d_w, d_lut, d_Wt, d_S);
        break;
    case REXSC_F16:
        expand_weight_kernel<__half><<<blocks, 256, 0, st>>>(a, (const __half *)d_w, d_lut, d_Wt, d_S);
        break;
    case REXSC_BF16:
        expand_weight_kernel<__nv_bfloat16><<<blocks, 256, 0, st>>>(a, (const __nv_bfloat16 *)d_w, d_lut, d_Wt, d_S);
        break;
    default: return REXSC_E_BAD_ARG;
    }
    REXSC_LAUNCH_CHECK("expand_weight_kernel");
    return REXSC_OK;
}

// ---- weight expansion straight to bit planes (operand format of the tensor-core kernel) ------------------------
// Wb[nchunk][slot][tap*CW + cw][row], row = sign*64 + local output channel, nibbles bit-reversed (the kernel's operand
// scaling).  One warp per (output channel, tap, channel word): lane = input channel; the 32 x 32 bit matrix
// (channel x slot) of each sign is transposed across the warp so that lane t holds slot t's channel-packed word.
__device__ __forceinline__ uint32_t transpose32_warp(uint32_t x, int lane)
{
    // recursive block swap across lanes: after the step with distance j, 2j x 2j blocks are transposed
#pragma unroll
    for (int j = 16; j >= 1; j >>= 1) {
        const uint32_t low = j == 16 ? 0x0000ffffu : j == 8 ? 0x00ff00ffu : j == 4 ? 0x0f0f0f0fu : j == 2 ? 0x33333333u : 0x55555555u;
        const uint32_t y = __shfl_xor_sync(0xffffffffu, x, j);
        x = (lane & j) ? ((x & ~low) | ((y & ~low) >> j)) : ((x & low) | ((y & low) << j));
    }
    return x;
}

__device__ __forceinline__ uint32_t reverse_nibbles(uint32_t v)
{
    v = __byte_perm(__brev(v), 0, 0x0123); // all 32 bits reversed, bytes back in order: every byte bit-reversed
    return ((v & 0x0f0f0f0fu) << 4) | ((v >> 4) & 0x0f0f0f0fu); // nibbles of a byte back in order
}

struct ExpandWBitsArgs {
    int C, Co, KH, KW, KHW, CW, NC;
    int period, nvals, words, linear_seeds, ohwi;
    float scale;
};

template <typename T>
__global__ void __launch_bounds__(256) expand_weight_bits_kernel(ExpandWBitsArgs a, const T *__restrict__ wt,
                                                                 const uint32_t *__restrict__ lut, uint32_t *__restrict__ Wb,
                                                                 long long items)
{
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int slots = a.words * 32;
    const size_t row_words = (size_t)a.KHW * a.CW;
    const long long item = (long long)blockIdx.x * 8 + warp;
    if (item >= items) return; // warp-uniform
    {
        const int cw = (int)(item % a.CW);
        long long t = item / a.CW;
        const int tap = (int)(t % a.KHW);
        const int co = (int)(t / a.KHW); // 0 .. NC*64: rows past Co stay zero
        const int kh = tap / a.KW, kw = tap - kh * a.KW;
        const int ci = cw * 32 + lane;
        int mag = 0;
        bool neg = false;
        if (ci < a.C && co < a.Co) {
            const long long wi = a.ohwi ? (((long long)co * a.KH + kh) * a.KW + kw) * a.C + ci
                                        : (((long long)co * a.C + ci) * a.KH + kh) * a.KW + kw;
            const float v = load_as_float<T>(wt, wi) * a.scale;
            // w_pos = ceil(clamp(v, 0, L-1)); w_neg = ceil(-clamp(v, 1-L, 0))  (sc_cuda.cpp:92-93)
            const int qp = (int)ceilf(fminf(fmaxf(v, 0.f), a.scale - 1.f));
            const int qn = (int)ceilf(-fminf(fmaxf(v, 1.f - a.scale), 0.f));
            if (qn > 0) { neg = true; mag = qn; } else { mag = qp; }
        }
        // seed index c*KH*KW + kh*KW + kw, offset 13 for both signs (sc_cuda_conv.cu:45,55-56); linear: c only
        const long long seed_ind = a.linear_seeds ? (long long)ci : ((long long)ci * a.KH + kh) * a.KW + kw;
        const int phase = (int)((13 + seed_ind) % a.period);
        const int nchunk = co >> 6, col = co & 63;
        for (int wd = 0; wd < a.words; wd++) {
            const uint32_t v = mag > 0 ? __ldg(lut + ((size_t)phase * a.nvals + mag) * a.words + wd) : 0u;
            const uint32_t tp = reverse_nibbles(transpose32_warp(neg ? 0u : v, lane));
            const uint32_t tn = reverse_nibbles(transpose32_warp(neg ? v : 0u, lane));
            uint32_t *dst = Wb + (((size_t)nchunk * slots + wd * 32 + lane) * row_words + (size_t)tap * a.CW + cw) * 128 + col;
            dst[0] = tp;
            dst[64] = tn;
        }
    }
}

int launch_expand_weight_bits(const ConvPlan &p, const rexsc_sc_conv_desc &d, const void *d_w, const uint32_t *d_lut,
                              uint32_t *d_Wb, cudaStream_t st)
{
    ExpandWBitsArgs a;
    a.C = p.C; a.Co = p.Co; a.KH = p.KH; a.KW = p.KW; a.KHW = p.KHW;
    a.CW = (p.C + 31) / 32; a.NC = (p.Co + 63) / 64;
    a.period = p.period; a.nvals = p.nvals; a.words = p.words; a.linear_seeds = d.linear_seeds;
    a.ohwi = d.w_channels_last; a.scale = (float)p.scale;
    const long long items = (long long)a.NC * 64 * a.KHW * a.CW;
    const long long blocks = (items + 7) / 8;
    if (blocks > 0x7fffffffLL) return REXSC_E_TOO_LONG;
    switch (d.w_dtype) {
    case REXSC_F32:
        expand_weight_bits_kernel<float><<<(unsigned)blocks, 256, 0, st>>>(a, (const float *)d_w, d_lut, d_Wb, items);
        break;
    case REXSC_F16:
        expand_weight_bits_kernel<__half><<<(unsigned)blocks, 256, 0, st>>>(a, (const __half *)d_w, d_lut, d_Wb, items);
        break;
    case REXSC_BF16:
        expand_weight_bits_kernel<__nv_bfloat16><<<(unsigned)blocks, 256, 0, st>>>(a, (const __nv_bfloat16 *)d_w, d_lut, d_Wb, items);
        break;
    default: return REXSC_E_BAD_ARG;
    }
    REXSC_LAUNCH_CHECK("expand_weight_bits_kernel");
    return REXSC_OK;
}

} // namespace rexsc
