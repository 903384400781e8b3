// Tiled SC conv forward for sm_100a: implicit GEMM over time-packed stream words on the integer ALU.
//
//   M = N*OH*OW output pixels, N = Cout, K = Cin*KH*KW; one 32-bit word per (element, 32 time slots).
//   CTA tile  = (32*TM) pixels x 32 output channels, NW warps (8 or 16).
//   Warp w owns TN = 32/NW output channels for ALL rows of the tile; lane owns rows lane + 32*j, j < TM.
//   Because every lane of a warp works on the same output channels at the same k, the sign of the weight
//   (which of the reference's two weight streams is non-zero) is warp-uniform: the kernel branches on it
//   and updates only the positive or only the negative accumulators, halving the LOP3 count.
//
//   Shared memory holds, per pipeline stage, the raw activation patch of 8 input channels
//   ([c][P - P_lo], P the stored pixel index of ConvPlan; the filter taps are address offsets into it, so
//   nothing is im2col-expanded, and columns are stored grouped by residue modulo the stride so that the lanes
//   of a warp read consecutive words for every tap at any stride) plus the 8-channel weight block and its sign words.  Stages are
//   filled by bulk async copies (cp.async.bulk, one per channel plane + two for the weights) issued by one
//   thread and tracked by an mbarrier; every wait on it is bounded and reports through a status word.
//
//   OR-n accumulation (torch_c/sc-extension/sc_device.cu:127-151, sc_device.cuh:338-340,380-384) as a
//   thermometer over 32 time slots at once:  x = a & w;  T_j |= T_{j-1} & x (j = n..2);  T_1 |= x;
//   result = sum_j popc(T_j) = sum_t min(count_t, n).  One launch handles one 32-slot word plane; longer
//   streams run one launch per plane and add into the int16 output.
#include "common.cuh"

namespace rexsc {

namespace {

constexpr int kStages = 2;
constexpr uint32_t kWaitLimit = 1u << 22; // bounded mbarrier polling (each poll may itself block briefly)

struct TiledArgs {
    int OH, OW, sh, sw, KH, KW, KHW, CCH, Co;
    int nrh, Wq, Hrows, Wrow, max_tap;
    long long M, NHWp;
    int out_nhwc, accumulate;
};

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count)
{
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes)
{
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
__device__ __forceinline__ bool mbar_try_wait(uint32_t bar, uint32_t parity)
{
    uint32_t ok;
    asm volatile(
        "{\n\t.reg .pred p;\n\t"
        "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
        "selp.u32 %0, 1, 0, p;\n\t}"
        : "=r"(ok)
        : "r"(bar), "r"(parity)
        : "memory");
    return ok != 0;
}
// Bounded wait: returns false (and the caller records it) instead of spinning for ever.
__device__ __forceinline__ bool mbar_wait_bounded(uint32_t bar, uint32_t parity)
{
    for (uint32_t i = 0; i < kWaitLimit; i++)
        if (mbar_try_wait(bar, parity)) return true;
    return false;
}
__device__ __forceinline__ void bulk_g2s(uint32_t dst, const void *src, uint32_t bytes, uint32_t bar)
{
    asm volatile("cp.async.bulk.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1], %2, [%3];" ::"r"(dst),
                 "l"(src), "r"(bytes), "r"(bar)
                 : "memory");
}

template <int NOR> __device__ __forceinline__ void thermo_update(uint32_t (&t)[NOR], uint32_t a, uint32_t w)
{
    const uint32_t x = a & w;
#pragma unroll
    for (int j = NOR - 1; j >= 1; j--) t[j] |= t[j - 1] & x;
    t[0] |= x;
}

template <int NOR, int TM, int NW>
__global__ void __launch_bounds__(NW * 32, 1)
sc_conv_tiled_kernel(TiledArgs a, const uint32_t *__restrict__ A, const uint32_t *__restrict__ Wt,
                     const uint32_t *__restrict__ S, int16_t *__restrict__ out_pos, int16_t *__restrict__ out_neg,
                     int *__restrict__ status)
{
    constexpr int BM = 32 * TM;
    constexpr int TN = kTileN / NW; // output channels per warp: 4 (8 warps) or 2 (16 warps)
    static_assert(TN == 2 || TN == 4, "warp tile is 2 or 4 output channels");
    extern __shared__ __align__(128) uint8_t smem[];
    const uint32_t a_stage_bytes = kChunkC * kPlaneWords * 4;
    const uint32_t b_stage_bytes = (uint32_t)a.KHW * kChunkC * kTileN * 4;
    const uint32_t s_stage_bytes = (uint32_t)a.KHW * (kTileN / kWarpN) * 4;
    uint8_t *a_base = smem;
    uint8_t *b_base = a_base + kStages * a_stage_bytes;
    uint8_t *s_base = b_base + kStages * b_stage_bytes;
    uint64_t *bars = reinterpret_cast<uint64_t *>(s_base + kStages * s_stage_bytes);
    int *tap_s = reinterpret_cast<int *>(bars + kStages); // word offset of every filter tap

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const int nt = blockIdx.x;                 // output-channel tile fastest: CTAs sharing a patch run together
    const uint32_t m0 = blockIdx.y * (uint32_t)BM; // first output pixel of the tile (M < 2^31, checked on the host)

    // stored pixel index of output pixel m at filter tap (0,0); fits 31 bits (NHWp < 2^31)
    auto pix0 = [&](uint32_t m) -> uint32_t {
        const uint32_t ow = m % (uint32_t)a.OW;
        const uint32_t t = m / (uint32_t)a.OW;
        const uint32_t oh = t % (uint32_t)a.OH;
        const uint32_t n = t / (uint32_t)a.OH;
        return (n * (uint32_t)a.Hrows + oh * (uint32_t)a.nrh) * (uint32_t)a.Wrow + ow;
    };
    const uint32_t m_last = (m0 + BM <= (uint32_t)a.M ? m0 + BM : (uint32_t)a.M) - 1;
    const uint32_t P_lo = pix0(m0) & ~3u;
    const uint32_t P_hi = pix0(m_last) + (uint32_t)a.max_tap;
    const uint32_t patch_words = ((P_hi - P_lo + 1) + 3) & ~3u;

    if (tid < a.KHW) {
        const int kh = tid / a.KW, kw = tid - kh * a.KW;
        tap_s[tid] = tap_offset(kh, kw, a.sh, a.sw, a.nrh, a.Wrow, a.Wq);
    }
    if (tid == 0) {
        for (int s = 0; s < kStages; s++) mbar_init(smem_u32(&bars[s]), 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    __syncthreads();

    const bool patch_ok = patch_words <= (uint32_t)kPlaneWords;
    bool failed = !patch_ok; // never true when the host-side fit check passed; guards the copies below

    auto issue = [&](int it) {
        const int s = it & 1;
        const uint32_t bar = smem_u32(&bars[s]);
        const uint32_t a_bytes = patch_words * 4;
        mbar_expect_tx(bar, kChunkC * a_bytes + b_stage_bytes + s_stage_bytes);
        const uint32_t *src = A + (size_t)it * kChunkC * a.NHWp + P_lo;
        const uint32_t dst = smem_u32(a_base + s * a_stage_bytes);
#pragma unroll
        for (int cc = 0; cc < kChunkC; cc++)
            bulk_g2s(dst + cc * kPlaneWords * 4, src + (size_t)cc * a.NHWp, a_bytes, bar);
        const size_t blk = ((size_t)nt * a.CCH + it) * a.KHW;
        bulk_g2s(smem_u32(b_base + s * b_stage_bytes), Wt + blk * (kChunkC * kTileN), b_stage_bytes, bar);
        bulk_g2s(smem_u32(s_base + s * s_stage_bytes), S + blk * (kTileN / kWarpN), s_stage_bytes, bar);
    };

    // first stage in flight while the per-row offsets are worked out
    int issued = 0;
    if (tid == 0 && !failed) {
        issue(0);
        issued = 1;
    }

    int off[TM];
#pragma unroll
    for (int j = 0; j < TM; j++) {
        uint32_t m = m0 + lane + 32 * j;
        if (m > m_last) m = m_last;
        off[j] = (int)(pix0(m) - P_lo);
    }

    uint32_t tp[TM][TN][NOR], tn[TM][TN][NOR];
#pragma unroll
    for (int j = 0; j < TM; j++)
#pragma unroll
        for (int c = 0; c < TN; c++)
#pragma unroll
            for (int q = 0; q < NOR; q++) { tp[j][c][q] = 0u; tn[j][c][q] = 0u; }

    for (int it = 0; it < a.CCH; it++) {
        const int s = it & 1;
        if (!failed) {
            if (!mbar_wait_bounded(smem_u32(&bars[s]), (uint32_t)((it >> 1) & 1))) failed = true;
        }
        // One barrier per step: every thread agrees on success, and everyone has finished reading the other
        // stage (step it-1), so it can be refilled for step it+1 while step it is computed.
        failed = __syncthreads_or(failed ? 1 : 0) != 0;
        if (failed) break;
        if (tid == 0 && it + 1 < a.CCH) { issue(it + 1); issued = it + 2; }

        const uint32_t *As = reinterpret_cast<const uint32_t *>(a_base + s * a_stage_bytes);
        const uint32_t *Bs = reinterpret_cast<const uint32_t *>(b_base + s * b_stage_bytes) + warp * TN;
        const uint32_t *Ss = reinterpret_cast<const uint32_t *>(s_base + s * s_stage_bytes) + (warp * TN) / kWarpN;
        const int sign_base = (warp * TN) % kWarpN; // first channel of this warp inside its 4-channel sign group

#pragma unroll 1
        for (int khw = 0; khw < a.KHW; khw++) {
            const int koff = tap_s[khw];
            const uint32_t sgw = Ss[khw * (kTileN / kWarpN)] >> sign_base;
            const uint32_t *ap[TM];
#pragma unroll
            for (int j = 0; j < TM; j++) ap[j] = As + off[j] + koff;
            const uint32_t *bp = Bs + khw * (kChunkC * kTileN);
#pragma unroll
            for (int cc = 0; cc < kChunkC; cc++) {
                uint32_t av[TM];
#pragma unroll
                for (int j = 0; j < TM; j++) av[j] = ap[j][cc * kPlaneWords];
                uint32_t wv[TN];
                if (TN == 4) {
                    const uint4 w4 = *reinterpret_cast<const uint4 *>(bp + cc * kTileN);
                    wv[0] = w4.x; wv[1] = w4.y; wv[TN - 2] = w4.z; wv[TN - 1] = w4.w;
                } else {
                    const uint2 w2 = *reinterpret_cast<const uint2 *>(bp + cc * kTileN);
                    wv[0] = w2.x; wv[1] = w2.y;
                }
#pragma unroll
                for (int c = 0; c < TN; c++) {
                    if (sgw & (1u << (cc * kWarpN + c))) {
#pragma unroll
                        for (int j = 0; j < TM; j++) thermo_update<NOR>(tn[j][c], av[j], wv[c]);
                    } else {
#pragma unroll
                        for (int j = 0; j < TM; j++) thermo_update<NOR>(tp[j][c], av[j], wv[c]);
                    }
                }
            }
        }
    }

    if (failed) {
        // report, then give copies that may still be in flight a bounded chance to land before exiting
        if (tid == 0) {
            atomicExch(status, patch_ok ? 1 : 2);
            // only the two most recent copies can still be in flight (one per stage)
            for (int it = issued > 2 ? issued - 2 : 0; it < issued; it++)
                (void)mbar_wait_bounded(smem_u32(&bars[it & 1]), (uint32_t)((it >> 1) & 1));
        }
        return;
    }

    // ---- epilogue: popcount the thermometers, store int16 in the requested layout -----------------
    const int co0 = nt * kTileN + warp * TN;
    const size_t ohw = (size_t)a.OH * a.OW;
#pragma unroll
    for (int j = 0; j < TM; j++) {
        const uint32_t m = m0 + lane + 32 * j;
        if (m > m_last) continue;
        int rp[TN], rn[TN];
#pragma unroll
        for (int c = 0; c < TN; c++) {
            rp[c] = 0; rn[c] = 0;
#pragma unroll
            for (int q = 0; q < NOR; q++) { rp[c] += __popc(tp[j][c][q]); rn[c] += __popc(tn[j][c][q]); }
        }
        if (a.out_nhwc) {
            const size_t base = (size_t)m * a.Co + co0;
            if ((a.Co & 3) == 0 && co0 + TN <= a.Co) {
                // TN consecutive int16 per row: one 4- or 8-byte store per output tensor
                uint32_t *pp = reinterpret_cast<uint32_t *>(out_pos + base);
                uint32_t *pn = reinterpret_cast<uint32_t *>(out_neg + base);
#pragma unroll
                for (int c = 0; c < TN; c += 2) {
                    if (a.accumulate) {
                        const uint32_t op = pp[c / 2], on = pn[c / 2];
                        rp[c] += (int16_t)(op & 0xffff); rp[c + 1] += (int16_t)(op >> 16);
                        rn[c] += (int16_t)(on & 0xffff); rn[c + 1] += (int16_t)(on >> 16);
                    }
                }
                if (TN == 4) {
                    uint2 vp, vn;
                    vp.x = (uint32_t)(rp[0] & 0xffff) | ((uint32_t)rp[1] << 16);
                    vp.y = (uint32_t)(rp[TN - 2] & 0xffff) | ((uint32_t)rp[TN - 1] << 16);
                    vn.x = (uint32_t)(rn[0] & 0xffff) | ((uint32_t)rn[1] << 16);
                    vn.y = (uint32_t)(rn[TN - 2] & 0xffff) | ((uint32_t)rn[TN - 1] << 16);
                    *reinterpret_cast<uint2 *>(pp) = vp;
                    *reinterpret_cast<uint2 *>(pn) = vn;
                } else {
                    pp[0] = (uint32_t)(rp[0] & 0xffff) | ((uint32_t)rp[1] << 16);
                    pn[0] = (uint32_t)(rn[0] & 0xffff) | ((uint32_t)rn[1] << 16);
                }
            } else {
#pragma unroll
                for (int c = 0; c < TN; c++) {
                    if (co0 + c < a.Co) {
                        if (a.accumulate) { rp[c] += out_pos[base + c]; rn[c] += out_neg[base + c]; }
                        out_pos[base + c] = (int16_t)rp[c];
                        out_neg[base + c] = (int16_t)rn[c];
                    }
                }
            }
        } else {
            const size_t pixel = (size_t)(m % (uint32_t)ohw);
            const size_t img = (size_t)(m / (uint32_t)ohw);
#pragma unroll
            for (int c = 0; c < TN; c++) {
                if (co0 + c < a.Co) {
                    const size_t oi = (img * a.Co + co0 + c) * ohw + pixel;
                    if (a.accumulate) { rp[c] += out_pos[oi]; rn[c] += out_neg[oi]; }
                    out_pos[oi] = (int16_t)rp[c];
                    out_neg[oi] = (int16_t)rn[c];
                }
            }
        }
    }
}

long long patch_bound(const ConvPlan &p, int BM)
{
    return patch_bound_words(BM, p.M, p.OW, p.OH, p.nrh, p.Hrows, p.Wrow, p.max_tap);
}

size_t tiled_smem_bytes(const ConvPlan &p)
{
    return (size_t)kStages * ((size_t)kChunkC * kPlaneWords * 4 + (size_t)p.KHW * kChunkC * kTileN * 4 +
                              (size_t)p.KHW * (kTileN / kWarpN) * 4) +
           kStages * sizeof(uint64_t) + kMaxKhw * sizeof(int);
}

// Tile shapes, best first, per OR-n.  16 warps x 2 channels keeps four warps per scheduler resident (the
// thermometer accumulators cap a 512-thread CTA at 128 registers per thread); OR-1 has so few LOP3 per loaded
// activation word that it keeps 4 channels per warp.
struct TileCfg { int tm, nw; };
int tile_candidates(int n_or, TileCfg (&out)[2])
{
    switch (n_or) {
    case 1: out[0] = {8, 8}; out[1] = {4, 8}; return 2;
    case 2: out[0] = {8, 16}; out[1] = {4, 16}; return 2;
    case 3: out[0] = {8, 16}; out[1] = {4, 16}; return 2; // 128 registers, a few bytes of spill
    default: out[0] = {4, 16}; return 1;
    }
}

bool pick_tile(const ConvPlan &p, TileCfg *cfg)
{
    TileCfg c[2];
    const int n = tile_candidates(p.n_or, c);
    for (int i = 0; i < n; i++)
        if (patch_bound(p, 32 * c[i].tm) <= kPlaneWords && (p.M + 32 * c[i].tm - 1) / (32 * c[i].tm) <= 65535) {
            *cfg = c[i];
            return true;
        }
    return false;
}

template <int NOR, int TM, int NW>
int launch_one(const ConvPlan &p, const TiledArgs &a, const uint32_t *A, const uint32_t *Wt, const uint32_t *S,
               int16_t *pos, int16_t *neg, int *status, cudaStream_t st)
{
    const size_t smem = tiled_smem_bytes(p);
    // per device and cheap: set on every launch rather than caching per process
    REXSC_CUDA_CHECK(cudaFuncSetAttribute(sc_conv_tiled_kernel<NOR, TM, NW>,
                                          cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    const long long tiles_m = (p.M + 32 * TM - 1) / (32 * TM);
    dim3 grid((unsigned)p.NT, (unsigned)tiles_m);
    sc_conv_tiled_kernel<NOR, TM, NW><<<grid, NW * 32, smem, st>>>(a, A, Wt, S, pos, neg, status);
    REXSC_LAUNCH_CHECK("sc_conv_tiled_kernel");
    return REXSC_OK;
}

} // namespace

bool conv_tiled_supported(const ConvPlan &p)
{
    if (p.n_or < 1 || p.n_or > 4) return false;
    if (p.KHW > kMaxKhw) return false;
    if (tiled_smem_bytes(p) > 227 * 1024) return false;
    TileCfg cfg;
    return pick_tile(p, &cfg);
}

int launch_conv_tiled(const ConvPlan &p, const rexsc_sc_conv_desc &d, const uint32_t *d_A, const uint32_t *d_Wt,
                      const uint32_t *d_S, int16_t *d_pos, int16_t *d_neg, int *d_status, cudaStream_t st)
{
    if (!conv_tiled_supported(p)) return REXSC_E_UNSUPPORTED;
    TiledArgs a;
    a.OH = p.OH; a.OW = p.OW; a.sh = p.sh; a.sw = p.sw;
    a.nrh = p.nrh; a.Wq = p.Wq; a.Hrows = p.Hrows; a.Wrow = p.Wrow; a.max_tap = p.max_tap;
    a.KH = p.KH; a.KW = p.KW; a.KHW = p.KHW; a.CCH = p.CCH; a.Co = p.Co;
    a.M = p.M; a.NHWp = p.NHWp; a.out_nhwc = d.out_channels_last;
    TileCfg cfg;
    pick_tile(p, &cfg);
    for (int wd = 0; wd < p.words; wd++) {
        a.accumulate = wd > 0;
        const uint32_t *A = d_A + (size_t)wd * p.a_plane_words;
        const uint32_t *Wt = d_Wt + (size_t)wd * p.w_plane_words;
        int rc = REXSC_E_UNSUPPORTED;
#define REXSC_TILED_CASE(NOR, TM, NW)                                                        \
    if (p.n_or == NOR && cfg.tm == TM && cfg.nw == NW)                                       \
        rc = launch_one<NOR, TM, NW>(p, a, A, Wt, d_S, d_pos, d_neg, d_status, st);
        REXSC_TILED_CASE(1, 8, 8)
        REXSC_TILED_CASE(1, 4, 8)
        REXSC_TILED_CASE(2, 8, 16)
        REXSC_TILED_CASE(2, 4, 16)
        REXSC_TILED_CASE(3, 8, 16)
        REXSC_TILED_CASE(3, 4, 16)
        REXSC_TILED_CASE(4, 4, 16)
#undef REXSC_TILED_CASE
        if (rc != REXSC_OK) return rc;
    }
    return REXSC_OK;
}

} // namespace rexsc
