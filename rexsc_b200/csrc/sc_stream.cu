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
    p->origin = 0;
    p->w_seed_pos = 13;
    p->w_seed_neg = 13;
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

bool make_compact_plan(const ConvPlan &p, ConvPlan *pc)
{
    if (!p.tc_ok || p.sh != 1 || p.sw != 1 || p.KH != 3 || p.KW != 3 || p.OH < 1 || p.OW < 1) return false;
    // the comparator works on int8: with 8-bit registers states above 127 read as negative and a zero VALUE still
    // produces ones, so a zero pixel's stream depends on its seed
    if (p.l > 7) return false;
    ConvPlan c = p;
    c.origin = 1;
    c.Hrows = p.OH + 1;
    c.Wq = p.OW + 1;
    c.Wrow = c.Wq; // no pitch padding: the flat stored index is the candidate index
    c.NHW = (long long)p.N * c.Hrows * c.Wrow;
    c.NHWp = (c.NHW + 3) / 4 * 4;
    c.a_plane_words = (long long)c.Cpad * c.NHWp;
    c.tc_ok = conv_tc_supported(c);
    if (!c.tc_ok || c.NHWp > p.NHWp) return false; // its planes live in the standard plan's region
    *pc = c;
    return true;
}

// ---- activation expansion -------------------------------------------------------------------
// Seed index of an activation element: c*Hp*Wp + h*Wp + w on the PADDED tensor, offset 0
// (torch_c/sc-extension/sc_cuda_conv.cu:133,139); linear: c only (sc_cuda_matmul.cu:177).
struct ExpandActArgs {
    int N, C, H, W, Hp, Wp, ph, pw, Cpad;
    int sh, sw, nrh, nrw, Wq, Hrows, Wrow;
    int origin;         // stored pixel (row', col') is padded pixel (h + origin, w + origin) of the mapping below
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
    h = (row / a.nrh) * a.sh + row % a.nrh + a.origin;
    w = (col % a.Wq) * a.sw + col / a.Wq + a.origin;
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
    a.sh = p.sh; a.sw = p.sw; a.nrh = p.nrh; a.nrw = p.nrw; a.Wq = p.Wq; a.Hrows = p.Hrows; a.Wrow = p.Wrow; a.origin = p.origin;
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

// ---- the same expansion for stream tables that fit shared memory twice over (stream lengths up to 64) -------------
// What the kernel above spends per element -- a byte load, the seed phase with its wrap-around, the table index, a
// select for zero values, 32-bit loads of single activations -- is cut down here so that the stage runs at memory speed:
//   * the table is kept in shared memory with its rows repeated once (phase rows 0 .. 2*period-2), so the phase of an
//     element, (channel part + pixel part), needs no modulo: index = pixel base + channel base + value * words + word,
//     one three-input add (plus one multiply-add when there is more than one word per stream);
//   * row `value 0` of the table is all zero (0 > state never holds), so padding, channels beyond C and zero activations
//     need no special case;
//   * channels_last inputs are read as 16-byte vectors (4 floats or 8 halves of one pixel per lane) and quantised
//     without a float-to-int conversion: clamp, add 2^23 rounding towards +inf, keep the low byte;
//   * the first two steps of the 32 x 32 bit transpose move whole bytes and are single byte-permute instructions;
//   * CTAs are persistent (the table is loaded once per CTA) and a warp handles all channel words of its 32 pixels, so
//     the pixel decode (three integer divisions) is paid once per 32 x C elements.
__device__ __forceinline__ uint32_t prmt(uint32_t a, uint32_t b, uint32_t sel)
{
    uint32_t r;
    asm("prmt.b32 %0, %1, %2, %3;" : "=r"(r) : "r"(a), "r"(b), "r"(sel));
    return r;
}
__device__ __forceinline__ void transpose32_regs_prmt(uint32_t (&v)[32])
{
#pragma unroll
    for (int k = 0; k < 16; k++) { // distance 16: half-words
        const uint32_t a = v[k], b = v[k + 16];
        v[k] = prmt(a, b, 0x5410u);
        v[k + 16] = prmt(a, b, 0x7632u);
    }
#pragma unroll
    for (int k = 0; k < 32; k++) { // distance 8: bytes
        if ((k & 8) == 0) {
            const uint32_t a = v[k], b = v[k + 8];
            v[k] = prmt(a, b, 0x6240u);
            v[k + 8] = prmt(a, b, 0x7351u);
        }
    }
#pragma unroll
    for (int j = 4; j >= 1; j >>= 1) {
        const uint32_t m = j == 4 ? 0x0f0f0f0fu : j == 2 ? 0x33333333u : 0x55555555u;
#pragma unroll
        for (int k = 0; k < 32; k++) {
            if ((k & j) == 0) {
                const uint32_t a = v[k], b = v[k + j];
                v[k] = (a & m) | ((b << j) & ~m);
                v[k + j] = ((a >> j) & m) | (b & ~m);
            }
        }
    }
}

// ceil(clamp(x * scale, 0, scale - 1)) as the low byte of a float: exact, because 0 <= v < 2^23 after the clamp and the
// addition rounds towards +infinity.  NaN inputs quantise to 0 like the comparison-based clamp of quant_ceil_unipolar.
__device__ __forceinline__ uint32_t quant_ceil_bits(float x, float scale, float top)
{
    const float v = fminf(fmaxf(x * scale, 0.f), top);
    return __float_as_uint(__fadd_ru(v, 8388608.0f));
}

template <typename T> struct ActVec;
template <> struct ActVec<float> {
    static constexpr int kElems = 4;
    static __device__ __forceinline__ uint32_t load_quant(const float *p, float scale, float top)
    {
        const float4 t = __ldg(reinterpret_cast<const float4 *>(p));
        const uint32_t lo = prmt(quant_ceil_bits(t.x, scale, top), quant_ceil_bits(t.y, scale, top), 0x0040u);
        const uint32_t hi = prmt(quant_ceil_bits(t.z, scale, top), quant_ceil_bits(t.w, scale, top), 0x0040u);
        return prmt(lo, hi, 0x5410u);
    }
};
template <> struct ActVec<__half> {
    static constexpr int kElems = 8;
    static __device__ __forceinline__ uint2 load_quant(const __half *p, float scale, float top)
    {
        const uint4 t = __ldg(reinterpret_cast<const uint4 *>(p));
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
        uint32_t b[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
            b[k] = prmt(quant_ceil_bits(f.x, scale, top), quant_ceil_bits(f.y, scale, top), 0x0040u);
        }
        return make_uint2(prmt(b[0], b[1], 0x5410u), prmt(b[2], b[3], 0x5410u));
    }
};
template <> struct ActVec<__nv_bfloat16> {
    static constexpr int kElems = 8;
    static __device__ __forceinline__ uint2 load_quant(const __nv_bfloat16 *p, float scale, float top)
    {
        const uint4 t = __ldg(reinterpret_cast<const uint4 *>(p));
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
        uint32_t b[4];
#pragma unroll
        for (int k = 0; k < 4; k++)
            b[k] = prmt(quant_ceil_bits(__uint_as_float(w[k] << 16), scale, top),
                        quant_ceil_bits(__uint_as_float(w[k] & 0xffff0000u), scale, top), 0x0040u);
        return make_uint2(prmt(b[0], b[1], 0x5410u), prmt(b[2], b[3], 0x5410u));
    }
};

__device__ __forceinline__ void store_bytes(uint32_t *dst, uint32_t v) { dst[0] = v; }
__device__ __forceinline__ void store_bytes(uint32_t *dst, uint2 v) { dst[0] = v.x; dst[1] = v.y; }

constexpr int kFastWarps = 8;
// VEC: channels_last input whose pixels' channel runs are 16-byte aligned (C a multiple of the vector width)
template <typename T, bool NHWC, bool VEC, int WORDS>
__global__ void __launch_bounds__(kFastWarps * 32, 2)
expand_act_bits_fast_kernel(ExpandActArgs a, const T *__restrict__ x, const uint32_t *__restrict__ lut_g,
                            uint32_t *__restrict__ Ab, int CW, long long n_groups)
{
    __shared__ __align__(16) uint8_t q_s[kFastWarps][32][44]; // [warp][pixel][channel]; the odd 11-word pitch puts the
                                                              // 32 lanes' rows into 32 different banks
    __shared__ long long xb_s[kFastWarps][32];                // [warp][pixel] input offset of the pixel's channel 0
    __shared__ uint32_t u_s[kFastWarps][32];                  // [warp][channel of the word] channel part of the index
    extern __shared__ __align__(16) uint32_t lut_s[];         // [2 * period - 1][nvals * words + 1]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const uint32_t period = (uint32_t)a.period;
    // one word of padding per row: the bank of an entry then depends on its phase as well, so the many lanes whose
    // activation is zero (same column of different rows) do not pile up on one bank
    const uint32_t row_src = (uint32_t)a.nvals * (uint32_t)WORDS, row_words = row_src + 1u;
    {
        const int rows = 2 * a.period - 1, all = rows * (int)row_src;
        for (int i = threadIdx.x; i < all; i += blockDim.x) {
            const int r = i / (int)row_src, col = i - r * (int)row_src;
            lut_s[r * (int)row_words + col] = __ldg(lut_g + (r < a.period ? r : r - a.period) * (int)row_src + col);
        }
        __syncthreads();
    }
    const float top = a.scale - 1.f;
    const size_t slot_stride = (size_t)CW * a.NHWp;
    for (long long grp = (long long)blockIdx.x * kFastWarps + warp; grp < n_groups; grp += (long long)gridDim.x * kFastWarps) {
        // lane = pixel: where it sits in the input
        const long long P0 = grp * 32, P = P0 + lane;
        int n = 0, h = 0, w = 0;
        const bool live = P < a.NHW && decode_pixel(a, P, n, h, w);
        const int hi = h - a.ph, wi = w - a.pw;
        const bool inside = live && hi >= 0 && hi < a.H && wi >= 0 && wi < a.W;
        const uint32_t pix_mod = a.linear_seeds ? 0u : ((uint32_t)h * (uint32_t)a.Wp + (uint32_t)w) % period;
        const uint32_t pix_base = pix_mod * row_words;
        const long long xbase = NHWC ? (((long long)n * a.H + hi) * a.W + wi) * a.C
                                     : (((long long)n * a.C) * a.H + hi) * a.W + wi;
        const bool store_ok = P < a.NHWp;
        if (NHWC) xb_s[warp][lane] = inside ? xbase : -1;
        for (int cw = 0; cw < CW; cw++) {
            const int c0 = cw * 32;
            __syncwarp(); // the previous word's tile has been consumed; xb_s is visible
            // ---- quantise the 32 pixels x 32 channels of this word into the byte tile ----
            if (NHWC && VEC) {
                constexpr int E = ActVec<T>::kElems, LPP = 32 / E, PPI = 32 / LPP; // lanes per pixel, pixels per pass
                const int ch = (lane % LPP) * E, pp = lane / LPP;
#pragma unroll
                for (int p0 = 0; p0 < 32; p0 += PPI) {
                    const long long xb = xb_s[warp][p0 + pp];
                    uint8_t *dst = &q_s[warp][p0 + pp][ch];
                    uint32_t *dst32 = reinterpret_cast<uint32_t *>(dst);
                    if (xb >= 0 && c0 + ch < a.C) {
                        store_bytes(dst32, ActVec<T>::load_quant(x + xb + c0 + ch, a.scale, top));
                    } else {
                        dst32[0] = 0u;
                        if (E == 8) dst32[1] = 0u;
                    }
                }
            } else if (NHWC) {
                const int c = c0 + lane;
                for (int p0 = 0; p0 < 32; p0++) {
                    const long long xb = xb_s[warp][p0];
                    const float val = (xb >= 0 && c < a.C) ? load_as_float<T>(x, xb + c) : 0.f;
                    q_s[warp][p0][lane] = (uint8_t)quant_ceil_bits(val, a.scale, top);
                }
            } else {
                const long long plane = (long long)a.H * a.W;
                constexpr int kBatch = 16;
#pragma unroll
                for (int cc0 = 0; cc0 < 32; cc0 += kBatch) {
                    float val[kBatch];
#pragma unroll
                    for (int i = 0; i < kBatch; i++) {
                        const int c = c0 + cc0 + i;
                        val[i] = (inside && c < a.C) ? load_as_float<T>(x, xbase + c * plane) : 0.f;
                    }
#pragma unroll
                    for (int i = 0; i < kBatch; i += 4) {
                        const uint32_t lo = prmt(quant_ceil_bits(val[i], a.scale, top), quant_ceil_bits(val[i + 1], a.scale, top), 0x0040u);
                        const uint32_t hi2 = prmt(quant_ceil_bits(val[i + 2], a.scale, top), quant_ceil_bits(val[i + 3], a.scale, top), 0x0040u);
                        *reinterpret_cast<uint32_t *>(&q_s[warp][lane][cc0 + i]) = prmt(lo, hi2, 0x5410u);
                    }
                }
            }
            // channel part of the table index for the 32 channels of this word (the same for every pixel)
            {
                const uint32_t c = (uint32_t)(c0 + lane);
                const uint32_t cph = a.linear_seeds ? c % period : (uint32_t)(((unsigned long long)c * a.plane_mod) % period);
                u_s[warp][lane] = cph * row_words;
            }
            __syncwarp();
            // ---- lane = pixel: look the 32 channels' stream words up, transpose, store 32 slot words ----
#pragma unroll
            for (int wd = 0; wd < WORDS; wd++) {
                uint32_t v[32];
#pragma unroll
                for (int c4 = 0; c4 < 32; c4 += 4) {
                    const uint32_t q4 = *reinterpret_cast<const uint32_t *>(&q_s[warp][lane][c4]);
                    const uint4 u4 = *reinterpret_cast<const uint4 *>(&u_s[warp][c4]);
                    const uint32_t uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const uint32_t q = (q4 >> (8 * k)) & 0xffu;
                        v[c4 + k] = lut_s[pix_base + uu[k] + (uint32_t)wd + q * (uint32_t)WORDS];
                    }
                }
                transpose32_regs_prmt(v);
                if (store_ok) {
                    uint32_t *dst = Ab + ((size_t)(wd * 32) * CW + cw) * a.NHWp + P;
#pragma unroll
                    for (int t = 0; t < 32; t++) {
                        __stcs(dst, v[t]);
                        dst += slot_stride;
                    }
                }
            }
        }
        __syncwarp();
    }
}

// ---- channels_last inputs with 16-byte aligned channel runs: the raw tile of the NEXT (pixel group, channel word) is
// fetched with cp.async into a per-warp staging buffer while the current one is quantised, looked up and transposed, so
// every warp keeps one tile of loads (4 KB of fp32) in flight all the time.  Without that the kernel above is latency-
// bound: its 16 warps per SM alternate between waiting for their loads and computing (ncu: issue slots 34 % busy,
// long_scoreboard the only stall that matters, DRAM 17 %).
__device__ __forceinline__ void cp_async16(void *smem_dst, const void *gmem_src, bool valid)
{
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 16 : 0; // 0: the 16 destination bytes are zero-filled, nothing is read
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async4(void *smem_dst, const void *gmem_src, bool valid)
{
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(smem_dst);
    const int bytes = valid ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(gmem_src), "r"(bytes) : "memory");
}
__device__ __forceinline__ void cp_async_commit() { asm volatile("cp.async.commit_group;" ::: "memory"); }
__device__ __forceinline__ void cp_async_wait_all_but_one() { asm volatile("cp.async.wait_group 1;" ::: "memory"); }

template <typename T> struct RawVec;
template <> struct RawVec<float> {
    static __device__ __forceinline__ uint32_t quant(const void *p, float scale, float top)
    {
        const float4 t = *reinterpret_cast<const float4 *>(p);
        const uint32_t lo = prmt(quant_ceil_bits(t.x, scale, top), quant_ceil_bits(t.y, scale, top), 0x0040u);
        const uint32_t hi = prmt(quant_ceil_bits(t.z, scale, top), quant_ceil_bits(t.w, scale, top), 0x0040u);
        return prmt(lo, hi, 0x5410u);
    }
};
template <> struct RawVec<__half> {
    static __device__ __forceinline__ uint2 quant(const void *p, float scale, float top)
    {
        const uint4 t = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
        uint32_t b[4];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
            b[k] = prmt(quant_ceil_bits(f.x, scale, top), quant_ceil_bits(f.y, scale, top), 0x0040u);
        }
        return make_uint2(prmt(b[0], b[1], 0x5410u), prmt(b[2], b[3], 0x5410u));
    }
};
template <> struct RawVec<__nv_bfloat16> {
    static __device__ __forceinline__ uint2 quant(const void *p, float scale, float top)
    {
        const uint4 t = *reinterpret_cast<const uint4 *>(p);
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
        uint32_t b[4];
#pragma unroll
        for (int k = 0; k < 4; k++)
            b[k] = prmt(quant_ceil_bits(__uint_as_float(w[k] << 16), scale, top),
                        quant_ceil_bits(__uint_as_float(w[k] & 0xffff0000u), scale, top), 0x0040u);
        return make_uint2(prmt(b[0], b[1], 0x5410u), prmt(b[2], b[3], 0x5410u));
    }
};

// Shared-memory scratch of the pipelined expansion, one set per warp
struct ActAsyncShared {
    uint8_t q[kFastWarps][32][44];     // [warp][pixel][channel] quantised values; odd 11-word pitch: 32 rows, 32 banks
    long long xb[kFastWarps][2][32];   // [warp][group buffer][pixel] input offset of the pixel's channel 0 (-1: padding)
    uint32_t u[kFastWarps][32];        // [warp][channel of the word] channel part of the table index
};

// The pipelined expansion of all groups of this CTA.  lut_s: the doubled, padded table, already in shared memory;
// raw_all: per warp (raw_stride bytes apart) two staging tiles of 32 pixels x 32 channels.
// NCHW: the staged tile is [channel][pixel].  fp32: fetched with 4-byte copies (one per channel and lane = pixel).
// 2-byte types (no 2-byte asynchronous copy exists): the next tile's 32 values per lane are loaded into registers
// before the current tile is processed and written to the other staging tile after it, which hides their latency the
// same way.
template <typename T, int WORDS, bool NCHW = false>
__device__ __forceinline__ void expand_act_async_body(const ExpandActArgs &a, const T *__restrict__ x,
                                                      const uint32_t *lut_s, uint8_t *raw_all, int raw_stride,
                                                      ActAsyncShared &sh, uint32_t *__restrict__ Ab, int CW,
                                                      long long n_groups)
{
    constexpr int E = 16 / (int)sizeof(T), LPP = 32 / E, PPI = 32 / LPP; // elements per lane, lanes per pixel, pixels per pass
    constexpr int kRowBytes = 32 * (int)sizeof(T), kTileBytes = 32 * kRowBytes;
    constexpr bool kRegStage = NCHW && sizeof(T) == 2; // staged through registers instead of cp.async
    uint32_t pre[kRegStage ? 16 : 1];                  // two 2-byte values per register: channels 2i, 2i + 1
    auto &q_s = sh.q;
    auto &xb_s = sh.xb;
    auto &u_s = sh.u;
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    uint8_t *raw_s = raw_all + (size_t)warp * raw_stride; // this warp's two staging tiles
    const uint32_t period = (uint32_t)a.period;
    const uint32_t row_src = (uint32_t)a.nvals * (uint32_t)WORDS, row_words = row_src + 1u;
    const float top = a.scale - 1.f;
    const size_t slot_stride = (size_t)CW * a.NHWp;
    const long long stride = (long long)gridDim.x * kFastWarps;
    const int ch = (lane % LPP) * E, pp = lane / LPP;

    struct Pix { long long P; uint32_t pix_base; bool store_ok; };
    // lane = pixel of group `grp`: input offset of its channel 0 into xb_s[warp][buf], seed phase and store position
    auto decode = [&](long long grp, int buf) {
        Pix r;
        r.P = grp * 32 + lane;
        int n = 0, h = 0, w = 0;
        const bool live = r.P < a.NHW && decode_pixel(a, r.P, n, h, w);
        const int hi = h - a.ph, wi = w - a.pw;
        const bool inside = live && hi >= 0 && hi < a.H && wi >= 0 && wi < a.W;
        const uint32_t pix_mod = a.linear_seeds ? 0u : ((uint32_t)h * (uint32_t)a.Wp + (uint32_t)w) % period;
        r.pix_base = pix_mod * row_words;
        r.store_ok = r.P < a.NHWp;
        xb_s[warp][buf][lane] = !inside ? -1
                                : NCHW  ? (((long long)n * a.C) * a.H + hi) * a.W + wi
                                        : (((long long)n * a.H + hi) * a.W + wi) * a.C;
        return r;
    };
    // start the copies of tile (group in xb_s[buf], channel word cw) into staging buffer `stage`
    // kRegStage: write the values that `issue` loaded into staging tile `stage`, [channel][pixel]
    auto land = [&](int stage) {
        if (!kRegStage) return;
        unsigned short *dst = reinterpret_cast<unsigned short *>(raw_s + stage * kTileBytes) + lane;
#pragma unroll
        for (int i = 0; i < (kRegStage ? 16 : 1); i++) {
            dst[(2 * i) * 32] = (unsigned short)(pre[i] & 0xffffu);
            dst[(2 * i + 1) * 32] = (unsigned short)(pre[i] >> 16);
        }
    };
    auto issue = [&](int buf, int cw, int stage) {
        uint8_t *dst = raw_s + stage * kTileBytes;
        if (kRegStage) {
            const long long xb = xb_s[warp][buf][lane], plane = (long long)a.H * a.W;
            const unsigned short *x16 = reinterpret_cast<const unsigned short *>(x);
#pragma unroll
            for (int i = 0; i < (kRegStage ? 16 : 1); i++) {
                const int c0 = cw * 32 + 2 * i;
                const uint32_t lo = (xb >= 0 && c0 < a.C) ? (uint32_t)__ldg(x16 + xb + c0 * plane) : 0u;
                const uint32_t hi = (xb >= 0 && c0 + 1 < a.C) ? (uint32_t)__ldg(x16 + xb + (c0 + 1) * plane) : 0u;
                pre[i] = lo | (hi << 16);
            }
            return;
        }
        if (NCHW) {
            const long long xb = xb_s[warp][buf][lane], plane = (long long)a.H * a.W;
#pragma unroll 8
            for (int cc = 0; cc < 32; cc++) {
                const bool ok = xb >= 0 && cw * 32 + cc < a.C;
                cp_async4(dst + cc * kRowBytes + lane * 4, ok ? (const void *)(x + xb + (cw * 32 + cc) * plane) : (const void *)x, ok);
            }
            cp_async_commit();
            return;
        }
        const int c = cw * 32 + ch;
#pragma unroll
        for (int p0 = 0; p0 < 32; p0 += PPI) {
            const long long xb = xb_s[warp][buf][p0 + pp];
            const bool ok = xb >= 0 && c < a.C;
            cp_async16(dst + (p0 + pp) * kRowBytes + ch * (int)sizeof(T), ok ? (const void *)(x + xb + c) : (const void *)x, ok);
        }
        cp_async_commit();
    };

    long long grp = (long long)blockIdx.x * kFastWarps + warp;
    if (grp >= n_groups) return; // warp-uniform; no block-wide barrier follows
    Pix cur = decode(grp, 0), nxt = cur;
    __syncwarp();
    issue(0, 0, 0);
    land(0);
    int buf = 0, stage = 0;
    for (;;) {
        const long long grp_next = grp + stride;
        const bool has_next = grp_next < n_groups;
        if (has_next) nxt = decode(grp_next, buf ^ 1);
        __syncwarp();
        for (int cw = 0; cw < CW; cw++) {
            // keep the next tile's loads in flight while this one is processed
            const bool more = cw + 1 < CW || has_next;
            if (cw + 1 < CW) issue(buf, cw + 1, stage ^ 1);
            else if (has_next) issue(buf ^ 1, 0, stage ^ 1);
            else if (!kRegStage) cp_async_commit(); // an empty group keeps the wait below uniform
            if (!kRegStage) cp_async_wait_all_but_one();
            __syncwarp();
            // ---- quantise the staged 32 pixels x 32 channels into the byte tile ----
            {
                const uint8_t *src = raw_s + stage * kTileBytes;
                if (NCHW) {
                    // lane = pixel reads its column of the [channel][pixel] tile and packs four channels per store
                    const T *colT = reinterpret_cast<const T *>(src) + lane;
                    auto col = [&](int c) { return load_as_float<T>(colT, (long long)c * 32); };
#pragma unroll
                    for (int c4 = 0; c4 < 32; c4 += 4) {
                        const uint32_t lo = prmt(quant_ceil_bits(col(c4), a.scale, top), quant_ceil_bits(col(c4 + 1), a.scale, top), 0x0040u);
                        const uint32_t hi2 = prmt(quant_ceil_bits(col(c4 + 2), a.scale, top), quant_ceil_bits(col(c4 + 3), a.scale, top), 0x0040u);
                        *reinterpret_cast<uint32_t *>(&q_s[warp][lane][c4]) = prmt(lo, hi2, 0x5410u);
                    }
                } else {
#pragma unroll
                    for (int p0 = 0; p0 < 32; p0 += PPI)
                        store_bytes(reinterpret_cast<uint32_t *>(&q_s[warp][p0 + pp][ch]),
                                    RawVec<T>::quant(src + (p0 + pp) * kRowBytes + ch * (int)sizeof(T), a.scale, top));
                }
                const uint32_t c = (uint32_t)(cw * 32 + lane);
                const uint32_t cph = a.linear_seeds ? c % period : (uint32_t)(((unsigned long long)c * a.plane_mod) % period);
                u_s[warp][lane] = cph * row_words;
            }
            __syncwarp();
            // ---- lane = pixel: look the 32 channels' stream words up, transpose, store 32 slot words ----
#pragma unroll
            for (int wd = 0; wd < WORDS; wd++) {
                uint32_t v[32];
#pragma unroll
                for (int c4 = 0; c4 < 32; c4 += 4) {
                    const uint32_t q4 = *reinterpret_cast<const uint32_t *>(&q_s[warp][lane][c4]);
                    const uint4 u4 = *reinterpret_cast<const uint4 *>(&u_s[warp][c4]);
                    const uint32_t uu[4] = {u4.x, u4.y, u4.z, u4.w};
#pragma unroll
                    for (int k = 0; k < 4; k++) {
                        const uint32_t q = (q4 >> (8 * k)) & 0xffu;
                        v[c4 + k] = lut_s[cur.pix_base + uu[k] + (uint32_t)wd + q * (uint32_t)WORDS];
                    }
                }
                transpose32_regs_prmt(v);
                if (cur.store_ok) {
                    uint32_t *dst = Ab + ((size_t)(wd * 32) * CW + cw) * a.NHWp + cur.P;
#pragma unroll
                    for (int t = 0; t < 32; t++) {
                        __stcs(dst, v[t]);
                        dst += slot_stride;
                    }
                }
            }
            __syncwarp(); // the byte tile, the index table and this staging buffer may be rewritten
            if (more) land(stage ^ 1);
            stage ^= 1;
        }
        if (!has_next) break;
        grp = grp_next;
        cur = nxt;
        buf ^= 1;
    }
}


// copy the global table into shared memory: rows repeated once, one word of padding per row
template <int WORDS>
__device__ __forceinline__ void load_doubled_table(const ExpandActArgs &a, const uint32_t *__restrict__ lut_g, uint32_t *lut_s)
{
    const int row_src = a.nvals * WORDS, row_words = row_src + 1;
    const int rows = 2 * a.period - 1, all = rows * row_src;
    for (int i = threadIdx.x; i < all; i += blockDim.x) {
        const int r = i / row_src, col = i - r * row_src;
        lut_s[r * row_words + col] = __ldg(lut_g + (r < a.period ? r : r - a.period) * row_src + col);
    }
}

template <typename T, int WORDS>
__global__ void __launch_bounds__(kFastWarps * 32, 2)
expand_act_bits_async_kernel(ExpandActArgs a, const T *__restrict__ x, const uint32_t *__restrict__ lut_g,
                             uint32_t *__restrict__ Ab, int CW, long long n_groups, int lut_smem_bytes)
{
    __shared__ __align__(16) ActAsyncShared sh;
    extern __shared__ __align__(16) uint32_t lut_s[]; // [2 * period - 1][nvals * words + 1], then the staging buffers
    load_doubled_table<WORDS>(a, lut_g, lut_s);
    __syncthreads();
    expand_act_async_body<T, WORDS>(a, x, lut_s, reinterpret_cast<uint8_t *>(lut_s) + lut_smem_bytes,
                                    2 * 32 * 32 * (int)sizeof(T), sh, Ab, CW, n_groups);
}

// helpers of the weight bit-plane expansion (used by the merged kernel below and by expand_weight_bits_kernel)
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
    int seed_pos, seed_neg; // ConvPlan::w_seed_pos / w_seed_neg
    float scale;
};

// ---- the whole expand stage of a tensor-core conv call in ONE launch ------------------------------------------------
// Stream tables, weight bit planes and activation bit planes used to be three dependent launches (plus the clearing of
// the status word); for the smaller layers their launch latencies, not their work, made up most of the stage.  Here
// every CTA builds both tables in its own shared memory straight from the LFSR (a few thousand short generator runs
// per CTA, nothing read from global memory), takes its share of the weight items, then runs the pipelined activation
// expansion.
// Table of stream words of every (seed phase, value), built in shared memory without running the generator per entry.
// Valid for gen_config 1 with progressive loading inactive (the front end's settings), where the activation and the
// weight table coincide.  The LFSR visits its states in one cycle c_0, c_1, ...; the generator seeded with state s emits
// at step t the comparison value > c_{pos(s) + t + 1}, so the word of (phase, value) has bit t set iff that threshold is
// below the value.  Per phase one thread scatters bit t into the entry `threshold + 1` of its (thread-private) row and
// then ORs the row's entries cumulatively: entry v ends up holding every bit whose threshold is < v.  Rows are written
// twice (phase and phase + period) with one word of padding, the layout the expansion kernels index without a modulo.
template <int WORDS>
__device__ __forceinline__ void build_doubled_table(const LutParams &lp, int period, int nvals, uint32_t *lut_s,
                                                    uint8_t *cyc_s, uint8_t *pos_s)
{
    const int row_words = nvals * WORDS + 1;
    if (threadIdx.x == 0) {
        int st = 1 - (lp.xnor ? 1 : 0);
        for (int k = 0; k < period; k++) {
            cyc_s[k] = (uint8_t)st;
            pos_s[st] = (uint8_t)k;
            st = lfsr_next(st, lp.l, lp.xnor);
        }
    }
    __syncthreads();
    for (int phase = threadIdx.x; phase < period; phase += blockDim.x) {
        uint32_t *row = lut_s + phase * row_words;
        for (int i = 0; i < nvals * WORDS; i++) row[i] = 0u;
        int k = pos_s[phase + 1 - (lp.xnor ? 1 : 0)];
        for (int t = 0; t < lp.bit_length; t++) {
            if (++k == period) k = 0;
            const int thr = cyc_s[k];
            if (thr + 1 < nvals) row[(thr + 1) * WORDS + (t >> 5)] |= 1u << (t & 31);
        }
        for (int v = 1; v < nvals; v++)
#pragma unroll
            for (int j = 0; j < WORDS; j++) row[v * WORDS + j] |= row[(v - 1) * WORDS + j];
    }
    __syncthreads();
    for (int i = threadIdx.x; i < (period - 1) * row_words; i += blockDim.x) lut_s[period * row_words + i] = lut_s[i];
    __syncthreads();
}

struct ExpandAllArgs {
    ExpandActArgs act;
    ExpandWBitsArgs w;
    LutParams lut;
    int w_dtype;
    int w_coarse;      // weight items are blocks of 32 output channels (else single output channels)
    long long w_items; // 0: activations only
    int verify_border; // check that the border pixels of the padded activation quantise to zero; status[1] = 1 otherwise
    int gate;          // run only if status[1] != 0
    int verify_vec;    // the border check may use 16-byte loads and 32-bit indices
};

__device__ __forceinline__ float load_weight_any(const void *w, int dtype, long long i)
{
    if (dtype == REXSC_F32) return static_cast<const float *>(w)[i];
    if (dtype == REXSC_F16) return __half2float(static_cast<const __half *>(w)[i]);
    return __bfloat162float(static_cast<const __nv_bfloat16 *>(w)[i]);
}

template <typename T, int WORDS, bool NCHW>
__global__ void __launch_bounds__(kFastWarps * 32, 2)
expand_all_kernel(ExpandAllArgs g, const T *__restrict__ x, const void *__restrict__ wt, uint32_t *__restrict__ Ab,
                  uint32_t *__restrict__ Wb, int *__restrict__ status, int CW, long long n_groups, int lut_smem_bytes)
{
    __shared__ __align__(16) ActAsyncShared sh;
    extern __shared__ __align__(16) uint32_t lut_s[];
    __shared__ uint8_t cyc_s[128], pos_s[128]; // the LFSR cycle and the position of every state in it
    const ExpandActArgs &a = g.act;
    if (g.gate && status[1] == 0) return; // fallback launch: the compact planes were valid, nothing to redo
    // the device status block of the workspace (when borders are verified the caller has cleared it: word 1 is being set)
    if (!g.verify_border && !g.gate && blockIdx.x == 0 && threadIdx.x < 64) status[threadIdx.x] = 0;
    if (g.verify_border) {
        // Every border pixel of the padded tensor (rows 0 and Hp-1, columns 0 and Wp-1) must quantise to zero, i.e. be
        // <= 0 (or NaN): the compact grid shares one zero row / column between neighbouring rows / images.
        const uint32_t per_img = 2u * (uint32_t)a.Wp + 2u * (uint32_t)(a.Hp - 2);
        auto border_pixel = [&](uint32_t b, int &hi, int &wi) { // b-th border pixel of an image -> input coordinates
            int h, w;
            if (b < (uint32_t)a.Wp) { h = 0; w = (int)b; }
            else if (b < 2u * (uint32_t)a.Wp) { h = a.Hp - 1; w = (int)b - a.Wp; }
            else { const int k = (int)b - 2 * a.Wp; h = 1 + (k >> 1); w = (k & 1) ? a.Wp - 1 : 0; }
            hi = h - a.ph; wi = w - a.pw;
            return hi >= 0 && hi < a.H && wi >= 0 && wi < a.W;
        };
        bool bad = false;
        constexpr int E = 16 / (int)sizeof(T);
        if (!NCHW && g.verify_vec) {
            // channels_last: 16 bytes of one pixel per load (32-bit index arithmetic, checked on the host)
            const uint32_t vecs = (uint32_t)a.C / E, total = (uint32_t)a.N * per_img * vecs;
#pragma unroll 4
            for (uint32_t idx = blockIdx.x * blockDim.x + threadIdx.x; idx < total; idx += gridDim.x * blockDim.x) {
                const uint32_t t = idx / vecs, v = idx - t * vecs, n = t / per_img, b = t - n * per_img;
                int hi, wi;
                if (border_pixel(b, hi, wi)) {
                    const uint4 raw = __ldg(reinterpret_cast<const uint4 *>(
                        x + (((size_t)n * a.H + hi) * a.W + wi) * a.C + (size_t)v * E));
                    const T *e = reinterpret_cast<const T *>(&raw);
#pragma unroll
                    for (int i = 0; i < E; i++) bad |= load_as_float<T>(e, i) > 0.f;
                }
            }
        } else {
            const long long total = (long long)a.N * per_img * a.C;
            for (long long idx = (long long)blockIdx.x * blockDim.x + threadIdx.x; idx < total;
                 idx += (long long)gridDim.x * blockDim.x) {
                // channel-planar: consecutive threads walk the border pixels of one channel
                const uint32_t b = (uint32_t)(idx % per_img);
                const long long t = idx / per_img;
                const int c = (int)(t % a.C), n = (int)(t / a.C);
                int hi, wi;
                if (border_pixel(b, hi, wi)) {
                    const long long xi = NCHW ? (((long long)n * a.C + c) * a.H + hi) * a.W + wi
                                              : (((long long)n * a.H + hi) * a.W + wi) * a.C + c;
                    bad |= load_as_float<T>(x, xi) > 0.f;
                }
            }
        }
        if (bad) atomicExch(status + 1, 1);
    }
    build_doubled_table<WORDS>(g.lut, a.period, a.nvals, lut_s, cyc_s, pos_s);
    // ---- weights: one warp per (block of 32 output channels, tap, channel word); lane = input channel of the word ----
    // For every output channel of the block the warp looks the 32 channels' stream words up and transposes them across
    // its lanes (lane = time slot afterwards); the 32 x 32 slot words of the block go through a swizzled tile in the
    // warp's staging area so that each slot's words leave as one 128-byte run over the output channels.
    {
        const ExpandWBitsArgs &wa = g.w;
        const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
        const int slots = WORDS * 32;
        const size_t row_words_w = (size_t)wa.KHW * wa.CW;
        const int row_words = wa.nvals * WORDS + 1;
        uint32_t *tile = reinterpret_cast<uint32_t *>(reinterpret_cast<uint8_t *>(lut_s) + lut_smem_bytes) + warp * 2048; // [2][32][32]
        // Small filters: one output channel per item (more items than warps matter more than coalesced stores).  The
        // weight of the warp's NEXT item is loaded before the current one is processed.
        auto fine_weight = [&](long long item) { // lane's weight of a fine item; 0 outside the tensor
            const int cw = (int)(item % wa.CW);
            const long long t = item / wa.CW;
            const int tap = (int)(t % wa.KHW), co = (int)(t / wa.KHW);
            const int kh = tap / wa.KW, kw = tap - kh * wa.KW;
            const int ci = cw * 32 + lane;
            if (item >= g.w_items || ci >= wa.C || co >= wa.Co) return 0.f;
            const long long wi = wa.ohwi ? (((long long)co * wa.KH + kh) * wa.KW + kw) * wa.C + ci
                                         : (((long long)co * wa.C + ci) * wa.KH + kh) * wa.KW + kw;
            return load_weight_any(wt, g.w_dtype, wi);
        };
        const long long item_step = (long long)gridDim.x * kFastWarps;
        float w_next = g.w_coarse ? 0.f : fine_weight((long long)blockIdx.x * kFastWarps + warp);
        for (long long item = (long long)blockIdx.x * kFastWarps + warp; !g.w_coarse && item < g.w_items; item += item_step) {
            const float w_cur = w_next;
            w_next = fine_weight(item + item_step);
            const int cw = (int)(item % wa.CW);
            long long t = item / wa.CW;
            const int tap = (int)(t % wa.KHW);
            const int co = (int)(t / wa.KHW); // 0 .. NC*64: rows past Co stay zero
            const int kh = tap / wa.KW, kw = tap - kh * wa.KW;
            const int ci = cw * 32 + lane;
            const float v = w_cur * wa.scale;
            // w_pos = ceil(clamp(v, 0, L-1)); w_neg = ceil(-clamp(v, 1-L, 0))  (sc_cuda.cpp:92-93)
            const int qp = (int)ceilf(fminf(fmaxf(v, 0.f), wa.scale - 1.f));
            const int qn = (int)ceilf(-fminf(fmaxf(v, 1.f - wa.scale), 0.f));
            const bool neg = qn > 0;
            const int mag = neg ? qn : qp;
            const long long seed_ind = wa.linear_seeds ? (long long)ci : ((long long)ci * wa.KH + kh) * wa.KW + kw;
            const int row_off = (int)(((neg ? wa.seed_neg : wa.seed_pos) + seed_ind) % wa.period) * row_words;
            const int nchunk = co >> 6, col = co & 63;
#pragma unroll
            for (int wd = 0; wd < WORDS; wd++) {
                const uint32_t v = lut_s[row_off + mag * WORDS + wd];
                uint32_t *dst = Wb + (((size_t)nchunk * slots + wd * 32 + lane) * row_words_w + (size_t)tap * wa.CW + cw) * 128 + col;
                dst[0] = reverse_nibbles(transpose32_warp(neg ? 0u : v, lane));
                dst[64] = reverse_nibbles(transpose32_warp(neg ? v : 0u, lane));
            }
        }
        // Large filters: 32 output channels per item, stores coalesced through the tile
        for (long long item = (long long)blockIdx.x * kFastWarps + warp; g.w_coarse && item < g.w_items;
             item += (long long)gridDim.x * kFastWarps) {
            const int cw = (int)(item % wa.CW);
            long long t = item / wa.CW;
            const int tap = (int)(t % wa.KHW);
            const int cb = (int)(t / wa.KHW); // block of 32 output channels, 0 .. 2*NC: rows past Co stay zero
            const int kh = tap / wa.KW, kw = tap - kh * wa.KW;
            const int ci = cw * 32 + lane;
            // seed index c*KH*KW + kh*KW + kw, offset 13 for both signs (sc_cuda_conv.cu:45,55-56); linear: c only
            const long long seed_ind = wa.linear_seeds ? (long long)ci : ((long long)ci * wa.KH + kh) * wa.KW + kw;
            const int row_off_pos = (int)((wa.seed_pos + seed_ind) % wa.period) * row_words;
            const int row_off_neg = (int)((wa.seed_neg + seed_ind) % wa.period) * row_words;
            const int nchunk = cb >> 1, col0 = (cb & 1) * 32;
#pragma unroll 1
            for (int wd = 0; wd < WORDS; wd++) {
                // eight output channels at a time: their loads are issued together, so the item costs four memory
                // latencies instead of thirty-two
#pragma unroll 1
                for (int cl0 = 0; cl0 < 32; cl0 += 8) {
                    float wv[8];
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int co = cb * 32 + cl0 + j;
                        wv[j] = 0.f;
                        if (ci < wa.C && co < wa.Co) {
                            const long long wi = wa.ohwi ? (((long long)co * wa.KH + kh) * wa.KW + kw) * wa.C + ci
                                                         : (((long long)co * wa.C + ci) * wa.KH + kh) * wa.KW + kw;
                            wv[j] = load_weight_any(wt, g.w_dtype, wi);
                        }
                    }
#pragma unroll
                    for (int j = 0; j < 8; j++) {
                        const int cl = cl0 + j;
                        const float v = wv[j] * wa.scale;
                        // w_pos = ceil(clamp(v, 0, L-1)); w_neg = ceil(-clamp(v, 1-L, 0))  (sc_cuda.cpp:92-93)
                        const int qp = (int)ceilf(fminf(fmaxf(v, 0.f), wa.scale - 1.f));
                        const int qn = (int)ceilf(-fminf(fmaxf(v, 1.f - wa.scale), 0.f));
                        const bool neg = qn > 0;
                        const int mag = neg ? qn : qp;
                        const uint32_t sw = lut_s[(neg ? row_off_neg : row_off_pos) + mag * WORDS + wd]; // row `value 0` is zero
                        tile[cl * 32 + (lane ^ cl)] = reverse_nibbles(transpose32_warp(neg ? 0u : sw, lane));
                        tile[1024 + cl * 32 + (lane ^ cl)] = reverse_nibbles(transpose32_warp(neg ? sw : 0u, lane));
                    }
                }
                __syncwarp();
                uint32_t *dst = Wb + (((size_t)nchunk * slots + wd * 32) * row_words_w + (size_t)tap * wa.CW + cw) * 128 + col0 + lane;
#pragma unroll 4
                for (int sl = 0; sl < 32; sl++) {
                    dst[0] = tile[lane * 32 + (sl ^ lane)];
                    dst[64] = tile[1024 + lane * 32 + (sl ^ lane)];
                    dst += row_words_w * 128;
                }
                __syncwarp();
            }
        }
    }
    // (each warp goes on as soon as its own weight items are done: its staging area is its own)
    expand_act_async_body<T, WORDS, NCHW>(a, x, lut_s, reinterpret_cast<uint8_t *>(lut_s) + lut_smem_bytes, 8192, sh, Ab, CW, n_groups);
}

template <typename T, int WORDS, bool NCHW>
static int launch_expand_all_t(const ExpandAllArgs &g, const void *d_act, const void *d_w, uint32_t *d_Ab, uint32_t *d_Wb,
                               int *d_status, int CW, size_t lut_bytes, cudaStream_t st)
{
    const long long n_groups = (g.act.NHWp + 31) / 32;
    int dev = 0, sms = 0;
    REXSC_CUDA_CHECK(cudaGetDevice(&dev));
    REXSC_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    long long blocks = (n_groups + kFastWarps - 1) / kFastWarps;
    const long long wblocks = (g.w_items + kFastWarps - 1) / kFastWarps;
    if (blocks < wblocks) blocks = wblocks;
    if (blocks > 2LL * sms) blocks = 2LL * sms; // persistent: two CTAs per SM
    const size_t lut_al = (lut_bytes + 15) / 16 * 16;
    // per warp: two activation tiles of 32 pixels x 32 channels, and at least the two 4 KB weight tiles
    const size_t staging = (size_t)kFastWarps * 8192;
    static_assert(2 * 32 * 32 * sizeof(T) <= 8192, "activation staging exceeds the per-warp area");
    auto kernel = expand_all_kernel<T, WORDS, NCHW>;
    REXSC_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)(lut_al + staging)));
    kernel<<<(unsigned)blocks, kFastWarps * 32, lut_al + staging, st>>>(g, (const T *)d_act, d_w, d_Ab, d_Wb, d_status, CW,
                                                                       n_groups, (int)lut_al);
    REXSC_LAUNCH_CHECK("expand_all_kernel");
    return REXSC_OK;
}

// The expand stage of the tensor-core path in one launch; REXSC_E_UNSUPPORTED when the shape does not qualify (the
// caller then uses the separate launches): channels_last activations with 16-byte aligned channel runs, at most two
// words per stream, tables that fit shared memory.
int launch_expand_all_bits(const ConvPlan &p, const rexsc_sc_conv_desc &d, const void *d_act, const void *d_w, int xnor,
                           uint32_t *d_Ab, uint32_t *d_Wb, int *d_status, const ExpandAllOptions &opt, cudaStream_t st)
{
    if ((p.words != 1 && p.words != 2) || p.NHWp >= (1LL << 31)) return REXSC_E_UNSUPPORTED;
    const int esz = d.act_dtype == REXSC_F32 ? 4 : 2;
    const bool nchw = !d.act_channels_last;
    if (nchw) {
        // channel-planar inputs are staged element by element: 4-byte copies (fp32) or plain 2-byte loads
        if ((reinterpret_cast<uintptr_t>(d_act) & (uintptr_t)(esz - 1)) != 0) return REXSC_E_UNSUPPORTED;
    } else if ((p.C % (16 / esz)) != 0 || (reinterpret_cast<uintptr_t>(d_act) & 15u) != 0) {
        return REXSC_E_UNSUPPORTED;
    }
    const size_t lut_bytes = (size_t)(2 * p.period - 1) * (p.nvals * p.words + 1) * sizeof(uint32_t);
    if (lut_bytes > 72 * 1024) return REXSC_E_UNSUPPORTED;
    // the in-kernel table builder covers the front end's generator settings: no AND-n replication, progressive loading
    // inactive (every value bit loaded from the first step on: load width - 1 >= total width)
    if (d.gen_config != 1 || d.prog_load_width - 1 < d.prog_total_width || p.l > 7) return REXSC_E_UNSUPPORTED;
    ExpandAllArgs g;
    ExpandActArgs &a = g.act;
    a.N = p.N; a.C = p.C; a.H = p.H; a.W = p.W; a.Hp = p.Hp; a.Wp = p.Wp; a.ph = p.ph; a.pw = p.pw;
    a.Cpad = p.Cpad; a.NHW = p.NHW; a.NHWp = p.NHWp; a.a_plane_words = p.a_plane_words;
    a.sh = p.sh; a.sw = p.sw; a.nrh = p.nrh; a.nrw = p.nrw; a.Wq = p.Wq; a.Hrows = p.Hrows; a.Wrow = p.Wrow; a.origin = p.origin;
    a.plane_mod = (uint32_t)(((long long)p.Hp * p.Wp) % p.period);
    a.period = p.period; a.nvals = p.nvals; a.words = p.words; a.linear_seeds = d.linear_seeds;
    a.scale = (float)p.scale;
    ExpandWBitsArgs &w = g.w;
    w.C = p.C; w.Co = p.Co; w.KH = p.KH; w.KW = p.KW; w.KHW = p.KHW;
    w.CW = (p.C + 31) / 32; w.NC = (p.Co + 63) / 64;
    w.period = p.period; w.nvals = p.nvals; w.words = p.words; w.linear_seeds = d.linear_seeds;
    w.ohwi = d.w_channels_last; w.scale = (float)p.scale;
    w.seed_pos = p.w_seed_pos; w.seed_neg = p.w_seed_neg;
    g.lut = LutParams{p.l, d.bit_length, d.gen_config, xnor, d.prog_total_width, d.prog_load_width, d.prog_load_wait, p.words};
    g.w_dtype = d.w_dtype;
    g.w_items = (long long)w.NC * 2 * w.KHW * w.CW; // blocks of 32 output channels x taps x channel words
    g.w_coarse = g.w_items >= 2048 ? 1 : 0;           // enough of them to occupy the grid's warps
    if (!g.w_coarse) g.w_items *= 32;                 // single output channels
    if (opt.skip_weights) g.w_items = 0;
    g.verify_border = opt.verify_border ? 1 : 0;
    g.gate = opt.gate ? 1 : 0;
    g.verify_vec = (!nchw && (long long)p.N * (2LL * p.Wp + 2LL * p.Hp) * p.C < (1LL << 31)) ? 1 : 0;
    const int CW = w.CW;
#define REXSC_ALL(T) (p.words == 1 ? launch_expand_all_t<T, 1, false>(g, d_act, d_w, d_Ab, d_Wb, d_status, CW, lut_bytes, st)   \
                                   : launch_expand_all_t<T, 2, false>(g, d_act, d_w, d_Ab, d_Wb, d_status, CW, lut_bytes, st))
#define REXSC_ALL_NCHW(T) (p.words == 1 ? launch_expand_all_t<T, 1, true>(g, d_act, d_w, d_Ab, d_Wb, d_status, CW, lut_bytes, st) \
                                        : launch_expand_all_t<T, 2, true>(g, d_act, d_w, d_Ab, d_Wb, d_status, CW, lut_bytes, st))
    if (nchw) {
        switch (d.act_dtype) {
        case REXSC_F32: return REXSC_ALL_NCHW(float);
        case REXSC_F16: return REXSC_ALL_NCHW(__half);
        case REXSC_BF16: return REXSC_ALL_NCHW(__nv_bfloat16);
        default: return REXSC_E_BAD_ARG;
        }
    }
#undef REXSC_ALL_NCHW
    switch (d.act_dtype) {
    case REXSC_F32: return REXSC_ALL(float);
    case REXSC_F16: return REXSC_ALL(__half);
    case REXSC_BF16: return REXSC_ALL(__nv_bfloat16);
    default: return REXSC_E_BAD_ARG;
    }
#undef REXSC_ALL
}

template <typename T, int WORDS>
static int launch_fast_t(const ExpandActArgs &a, bool nhwc, const void *d_act, const uint32_t *d_lut, uint32_t *d_Ab,
                         int CW, size_t lut_bytes, cudaStream_t st)
{
    const long long n_groups = (a.NHWp + 31) / 32;
    int dev = 0, sms = 0;
    REXSC_CUDA_CHECK(cudaGetDevice(&dev));
    REXSC_CUDA_CHECK(cudaDeviceGetAttribute(&sms, cudaDevAttrMultiProcessorCount, dev));
    long long blocks = (n_groups + kFastWarps - 1) / kFastWarps;
    if (blocks > 2LL * sms) blocks = 2LL * sms; // persistent: two CTAs per SM, each loads the table once
    constexpr int E = 16 / (int)sizeof(T);
    const bool vec = nhwc && (a.C % E) == 0 && (reinterpret_cast<uintptr_t>(d_act) & 15u) == 0;
    auto run = [&](auto kernel) -> int {
        REXSC_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)lut_bytes));
        kernel<<<(unsigned)blocks, kFastWarps * 32, lut_bytes, st>>>(a, (const T *)d_act, d_lut, d_Ab, CW, n_groups);
        REXSC_LAUNCH_CHECK("expand_act_bits_fast_kernel");
        return REXSC_OK;
    };
    if (!nhwc) return run(expand_act_bits_fast_kernel<T, false, false, WORDS>);
    if (vec) {
        // staging: two tiles of 32 pixels x 32 channels per warp behind the table
        const size_t lut_al = (lut_bytes + 15) / 16 * 16;
        const size_t smem = lut_al + (size_t)kFastWarps * 2 * 32 * 32 * sizeof(T);
        auto kernel = expand_act_bits_async_kernel<T, WORDS>;
        REXSC_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
        kernel<<<(unsigned)blocks, kFastWarps * 32, smem, st>>>(a, (const T *)d_act, d_lut, d_Ab, CW, n_groups, (int)lut_al);
        REXSC_LAUNCH_CHECK("expand_act_bits_async_kernel");
        return REXSC_OK;
    }
    return run(expand_act_bits_fast_kernel<T, true, false, WORDS>);
}

static int launch_expand_act_bits_fast(const ExpandActArgs &a, const rexsc_sc_conv_desc &d, bool nhwc, const void *d_act,
                                       const uint32_t *d_lut, uint32_t *d_Ab, int CW, size_t lut_bytes, cudaStream_t st)
{
#define REXSC_FAST(T) (a.words == 1 ? launch_fast_t<T, 1>(a, nhwc, d_act, d_lut, d_Ab, CW, lut_bytes, st)             \
                                    : launch_fast_t<T, 2>(a, nhwc, d_act, d_lut, d_Ab, CW, lut_bytes, st))
    switch (d.act_dtype) {
    case REXSC_F32: return REXSC_FAST(float);
    case REXSC_F16: return REXSC_FAST(__half);
    case REXSC_BF16: return REXSC_FAST(__nv_bfloat16);
    default: return REXSC_E_BAD_ARG;
    }
#undef REXSC_FAST
}

int launch_expand_act_bits(const ConvPlan &p, const rexsc_sc_conv_desc &d, const void *d_act, const uint32_t *d_lut,
                           uint32_t *d_Ab, cudaStream_t st)
{
    ExpandActArgs a;
    a.N = p.N; a.C = p.C; a.H = p.H; a.W = p.W; a.Hp = p.Hp; a.Wp = p.Wp; a.ph = p.ph; a.pw = p.pw;
    a.Cpad = p.Cpad; a.NHW = p.NHW; a.NHWp = p.NHWp; a.a_plane_words = p.a_plane_words;
    a.sh = p.sh; a.sw = p.sw; a.nrh = p.nrh; a.nrw = p.nrw; a.Wq = p.Wq; a.Hrows = p.Hrows; a.Wrow = p.Wrow; a.origin = p.origin;
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
    const size_t fast_lut_bytes = (size_t)(2 * p.period - 1) * (p.nvals * p.words + 1) * sizeof(uint32_t);
    if ((p.words == 1 || p.words == 2) && fast_lut_bytes <= 72 * 1024 && p.NHWp < (1LL << 31))
        return launch_expand_act_bits_fast(a, d, nhwc, d_act, d_lut, d_Ab, CW, fast_lut_bytes, st);
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
    int seed_pos, seed_neg; // ConvPlan::w_seed_pos / w_seed_neg
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
    int phase = (int)(((neg ? a.seed_neg : a.seed_pos) + seed_ind) % a.period);
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
    a.seed_pos = p.w_seed_pos; a.seed_neg = p.w_seed_neg;
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
        const int phase = (int)(((neg ? a.seed_neg : a.seed_pos) + seed_ind) % a.period);
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
    a.seed_pos = p.w_seed_pos; a.seed_neg = p.w_seed_neg;
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
