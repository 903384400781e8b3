// Direct SC conv forward: one thread per output element, operands read straight from global memory.
// It accepts every shape and every OR-n the library supports and is the fallback of the tiled kernel
// (and the second opinion its results are compared with in the tests).
//
// Arithmetic (torch_c/sc-extension/sc_device.cu:127-151, sc_device.cuh:338-340,380-384):
//   out = sum over time slots of min(count_slot, n),  count_slot = sum_k a_bit & w_bit
// With time-packed words (bit t = slot t) the saturating count is kept as a thermometer
// T_j = "count >= j in this slot": x = a & w;  T_j |= T_{j-1} & x (j = n..2);  T_1 |= x;
// and out = sum_j popc(T_j).  For n > 4 a 16-plane bit-sliced binary counter is used instead and
// min(count, n) is applied per slot at the end.
#include "common.cuh"

namespace rexsc {

struct DirectArgs {
    int OH, OW, sh, sw, KH, KW, KHW, CCH, NT, Co, words, n_or;
    int nrh, Wq, Hrows, Wrow;
    long long M, NHWp, a_plane_words, w_plane_words;
    int out_nhwc;
};

template <int NOR>
__global__ void __launch_bounds__(256) sc_conv_direct_kernel(DirectArgs a, const uint32_t *__restrict__ A,
                                                             const uint32_t *__restrict__ Wt,
                                                             const uint32_t *__restrict__ S,
                                                             int16_t *__restrict__ out_pos,
                                                             int16_t *__restrict__ out_neg)
{
    // block = 32 output channels (x) x 8 output pixels (y)
    const int nl = threadIdx.x & 31;
    const int my = threadIdx.x >> 5;
    const long long m = (long long)blockIdx.x * 8 + my;
    const int nt = blockIdx.y;
    const int co = nt * kTileN + nl;
    if (m >= a.M) return;
    const int ow = (int)(m % a.OW);
    const long long t = m / a.OW;
    const int oh = (int)(t % a.OH);
    const int n = (int)(t / a.OH);
    const long long P0 = ((long long)n * a.Hrows + (long long)oh * a.nrh) * a.Wrow + ow;
    const int w8 = nl >> 2, col = nl & 3;

    int res_pos = 0, res_neg = 0;
    for (int wd = 0; wd < a.words; wd++) {
        const uint32_t *Aw = A + (size_t)wd * a.a_plane_words;
        const uint32_t *Ww = Wt + (size_t)wd * a.w_plane_words;
        uint32_t tp[NOR > 0 ? NOR : 16], tn[NOR > 0 ? NOR : 16];
#pragma unroll
        for (int j = 0; j < (NOR > 0 ? NOR : 16); j++) { tp[j] = 0u; tn[j] = 0u; }
        for (int cch = 0; cch < a.CCH; cch++) {
            for (int khw = 0; khw < a.KHW; khw++) {
                const int kh = khw / a.KW, kw = khw - kh * a.KW;
                const int tap = tap_offset(kh, kw, a.sh, a.sw, a.nrh, a.Wrow, a.Wq);
                const size_t blk = ((size_t)nt * a.CCH + cch) * a.KHW + khw;
                const uint32_t sg = __ldg(S + blk * 8 + w8);
#pragma unroll
                for (int cc = 0; cc < kChunkC; cc++) {
                    const int c = cch * kChunkC + cc;
                    const uint32_t av = __ldg(Aw + (size_t)c * a.NHWp + P0 + tap);
                    const uint32_t wv = __ldg(Ww + (blk * kChunkC + cc) * kTileN + nl);
                    uint32_t x = av & wv;
                    const bool neg = (sg >> (cc * 4 + col)) & 1u;
                    uint32_t xp = neg ? 0u : x, xn = neg ? x : 0u;
                    if (NOR > 0) {
#pragma unroll
                        for (int j = NOR - 1; j >= 1; j--) {
                            tp[j] |= tp[j - 1] & xp;
                            tn[j] |= tn[j - 1] & xn;
                        }
                        tp[0] |= xp;
                        tn[0] |= xn;
                    } else {
                        // ripple-carry add of a 1-bit-per-slot word into 16 counter planes
#pragma unroll
                        for (int j = 0; j < 16; j++) {
                            uint32_t cp = tp[j] & xp;
                            tp[j] ^= xp;
                            xp = cp;
                            uint32_t cn = tn[j] & xn;
                            tn[j] ^= xn;
                            xn = cn;
                        }
                    }
                }
            }
        }
        if (NOR > 0) {
#pragma unroll
            for (int j = 0; j < NOR; j++) {
                res_pos += __popc(tp[j]);
                res_neg += __popc(tn[j]);
            }
        } else {
            for (int b = 0; b < 32; b++) {
                int cp = 0, cn = 0;
#pragma unroll
                for (int j = 0; j < 16; j++) {
                    cp |= (int)((tp[j] >> b) & 1u) << j;
                    cn |= (int)((tn[j] >> b) & 1u) << j;
                }
                res_pos += min(cp, a.n_or);
                res_neg += min(cn, a.n_or);
            }
        }
    }
    if (co < a.Co) {
        size_t oi = a.out_nhwc ? (size_t)m * a.Co + co
                               : ((size_t)n * a.Co + co) * ((size_t)a.OH * a.OW) + (size_t)oh * a.OW + ow;
        out_pos[oi] = (int16_t)res_pos;
        out_neg[oi] = (int16_t)res_neg;
    }
}

int launch_conv_direct(const ConvPlan &p, const rexsc_sc_conv_desc &d, const uint32_t *d_A, const uint32_t *d_Wt,
                       const uint32_t *d_S, int16_t *d_pos, int16_t *d_neg, cudaStream_t st)
{
    DirectArgs a;
    a.OH = p.OH; a.OW = p.OW; a.sh = p.sh; a.sw = p.sw;
    a.nrh = p.nrh; a.Wq = p.Wq; a.Hrows = p.Hrows; a.Wrow = p.Wrow;
    a.KH = p.KH; a.KW = p.KW; a.KHW = p.KHW; a.CCH = p.CCH; a.NT = p.NT; a.Co = p.Co;
    a.words = p.words; a.n_or = p.n_or; a.M = p.M; a.NHWp = p.NHWp;
    a.a_plane_words = p.a_plane_words; a.w_plane_words = p.w_plane_words;
    a.out_nhwc = d.out_channels_last;
    dim3 grid((unsigned)((p.M + 7) / 8), (unsigned)p.NT);
    if (grid.y > 65535) return REXSC_E_TOO_LONG;
    switch (p.n_or <= 4 ? p.n_or : 0) {
    case 1: sc_conv_direct_kernel<1><<<grid, 256, 0, st>>>(a, d_A, d_Wt, d_S, d_pos, d_neg); break;
    case 2: sc_conv_direct_kernel<2><<<grid, 256, 0, st>>>(a, d_A, d_Wt, d_S, d_pos, d_neg); break;
    case 3: sc_conv_direct_kernel<3><<<grid, 256, 0, st>>>(a, d_A, d_Wt, d_S, d_pos, d_neg); break;
    case 4: sc_conv_direct_kernel<4><<<grid, 256, 0, st>>>(a, d_A, d_Wt, d_S, d_pos, d_neg); break;
    default: sc_conv_direct_kernel<0><<<grid, 256, 0, st>>>(a, d_A, d_Wt, d_S, d_pos, d_neg); break;
    }
    REXSC_LAUNCH_CHECK("sc_conv_direct_kernel");
    return REXSC_OK;
}

} // namespace rexsc
