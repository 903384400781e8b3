// Shared declarations of the rexsc_b200 CUDA library (sm_100a only).
#pragma once

#include <cuda_bf16.h>
#include <cuda_fp16.h>
#include <cuda_runtime.h>
#include <stdint.h>

#include "../../include/rexsc_b200.h"

namespace rexsc {

// ---- error plumbing -------------------------------------------------------------------------
void set_cuda_error(cudaError_t e, const char *where);
// every kernel launch of the library is followed by exactly one REXSC_LAUNCH_CHECK, which counts it
// (rexsc_kernel_launch_count)
void note_kernel_launch();
#define REXSC_CUDA_CHECK(expr)                                  \
    do {                                                        \
        cudaError_t _e = (expr);                                \
        if (_e != cudaSuccess) {                                \
            ::rexsc::set_cuda_error(_e, #expr);                 \
            return REXSC_E_CUDA;                                \
        }                                                       \
    } while (0)
#define REXSC_LAUNCH_CHECK(what)                                \
    do {                                                        \
        ::rexsc::note_kernel_launch();                          \
        cudaError_t _e = cudaGetLastError();                    \
        if (_e != cudaSuccess) {                                \
            ::rexsc::set_cuda_error(_e, what);                  \
            return REXSC_E_CUDA;                                \
        }                                                       \
    } while (0)

// ---- geometry of the tiled SC conv kernel (shared by the weight packer and the kernel) -------
constexpr int kChunkC = 8;        // input channels staged per pipeline step
constexpr int kTileN = 32;        // output channels per CTA
constexpr int kWarpN = 4;         // output channels per warp (8 warps x 4 = kTileN)
constexpr int kPlaneWords = 1536; // shared-memory words per staged channel plane (patch capacity)
constexpr int kMaxKhw = 49;       // largest filter footprint the tiled kernel stages (7x7)

static inline size_t align_up(size_t v, size_t a) { return (v + a - 1) / a * a; }

// Everything the kernels need to know about one SC conv call, derived on the host.
struct ConvPlan {
    // generator
    int l;         // LFSR length in bits
    int period;    // 2^l - 1
    int nvals;     // 2^l
    int scale;     // quantisation scale of activations and weights: 2^l when the caller gives the LFSR length,
                   // else bit_length (sc_cuda.cpp:76-77,90-91; differs from 2^l only for bit_length 2 and 4)
    int slots;     // bit_length * gen_config
    int words;     // ceil(slots / 32)
    int n_or;      // OR-n limit (bin_config + 1)
    // geometry
    int N, C, H, W;       // activation before padding
    int Hp, Wp;           // after the op's own padding
    int Co, KH, KW, KHW;
    int OH, OW;
    int sh, sw, ph, pw;
    // Stored pixel grid of the activation words.  Only rows / columns a filter tap can touch are kept, and
    // columns are grouped by their residue modulo the stride so that consecutive output pixels read
    // consecutive words for every tap (stride 1: the plain padded grid):
    //   row'  = (h / sh) * nrh + h % sh      kept iff h % sh < nrh = min(sh, KH)
    //   col'  = (w % sw) * Wq + w / sw       kept iff w % sw < nrw = min(sw, KW),  Wq = ceil(Wp / sw)
    //   P     = (n * Hrows + row') * Wrow + col',   Hrows = ceil(Hp / sh) * nrh,  Wrow = Wq * nrw
    int nrh, nrw, Wq, Hrows, Wrow;
    // seed offsets of the weight generators: the phase of a weight is (offset + seed index) mod period, per sign.  The
    // extension seeds both signs at 13 (sc_cuda_conv.cu:45,55-56; sc_cuda_matmul.cu:77-78); the front end's pure-torch
    // linear bit loop seeds positive weights at 67 and negative ones at 37 (utils_functional.py:147-165).
    int w_seed_pos, w_seed_neg;
    int origin;           // 0: stored pixel (row', col') as above.  1: compact grid of 3x3 stride-1 layers whose border
                          // pixels are zero (see make_compact_plan): stored pixel (r, c) = padded pixel (r + 1, c + 1)
    int max_tap;          // largest tap offset (see tap_offset)
    long long NHW;        // N * Hrows * Wrow
    long long NHWp;       // plane stride of the activation words (multiple of 4)
    long long M;          // N * OH * OW
    int Cpad, CCH;        // c_in padded to kChunkC, number of channel chunks
    int NT;               // ceil(Co / kTileN)
    long long Kdot;       // C * KH * KW, length of the dot product
    // workspace layout (byte offsets)
    size_t off_status, off_lut_a, off_lut_w, off_A, off_Wt, off_S, off_tc, total;
    bool tc_ok;           // the tensor-core kernel can run this shape (its bit planes live at off_tc)
    // per-plane sizes in words
    long long a_plane_words; // Cpad * NHWp  (one stream-word plane of activations)
    long long w_plane_words; // NT * CCH * KHW * kChunkC * kTileN
};

int make_conv_plan(const rexsc_sc_conv_desc *d, ConvPlan *p);

// Compact activation grid for the tensor-core path of 3x3 stride-1 layers whose zero border is one pixel wide (what
// padding 1 produces).  The standard grid stores every padded pixel, Hp x Wp per image, and the tensor-core kernel
// computes one candidate row per stored pixel; (Hp*Wp - OH*OW) / (Hp*Wp) of them are no output pixel (40 % on 7x7
// maps).  If all four border rows / columns are zero, one zero column can serve as the right border of a row AND the
// left border of the next row, and one zero row as the bottom border of an image AND the top border of the next:
// per image (OH + 1) x (OW + 1) stored pixels and candidates, stored pixel (r, c) = padded pixel (r + 1, c + 1), output
// (i, j) centred on stored pixel (i, j), tap (kh, kw) at flat offset (kh - 1) * (OW + 1) + (kw - 1).  Zero pixels have
// all-zero streams whatever their seed, so sharing them changes no count.  Returns false when the layer does not
// qualify; *pc is then untouched.
bool make_compact_plan(const ConvPlan &p, ConvPlan *pc);

// Word offset of filter tap (kh, kw) relative to the word of tap (0, 0) of the same output pixel.
__host__ __device__ __forceinline__ int tap_offset(int kh, int kw, int sh, int sw, int nrh, int Wrow, int Wq)
{
    return ((kh / sh) * nrh + kh % sh) * Wrow + (kw % sw) * Wq + kw / sw;
}

// ---- host launchers (each enqueues on `st`, returns REXSC_*) -----------------------------------
int launch_build_lut(int l, int bit_length, int gen_config, int xnor, int tw, int lw, int lwait, int is_weight,
                     uint32_t *d_lut, cudaStream_t st);
int launch_expand_act(const ConvPlan &p, const rexsc_sc_conv_desc &d, const void *d_act, const uint32_t *d_lut,
                      uint32_t *d_A, cudaStream_t st);
// the same expansion, written as channel-packed bit planes Ab[slot][cw][P] for the tensor-core kernel
int launch_expand_act_bits(const ConvPlan &p, const rexsc_sc_conv_desc &d, const void *d_act, const uint32_t *d_lut,
                           uint32_t *d_Ab, cudaStream_t st);
int launch_expand_weight(const ConvPlan &p, const rexsc_sc_conv_desc &d, const void *d_w, const uint32_t *d_lut,
                         uint32_t *d_Wt, uint32_t *d_S, cudaStream_t st);
int launch_conv_direct(const ConvPlan &p, const rexsc_sc_conv_desc &d, const uint32_t *d_A, const uint32_t *d_Wt,
                       const uint32_t *d_S, int16_t *d_pos, int16_t *d_neg, cudaStream_t st);
bool conv_tiled_supported(const ConvPlan &p);
int launch_conv_tiled(const ConvPlan &p, const rexsc_sc_conv_desc &d, const uint32_t *d_A, const uint32_t *d_Wt,
                      const uint32_t *d_S, int16_t *d_pos, int16_t *d_neg, int *d_status, cudaStream_t st);

// Upper bound of the activation patch (in words per channel plane) a tile of BM output pixels can need in the
// tiled kernel's shared-memory stage, for a given stored-grid geometry.
static inline long long patch_bound_words(long long BM, long long M, int OW, int OH, int nrh, int Hrows, int Wrow,
                                          int max_tap)
{
    if (BM > M) BM = M;                              // a tile never holds more pixels than exist
    const long long dR = (BM + OW - 2) / OW;         // output-row boundaries a tile can cross
    const long long dI = (dR + OH - 1) / OH;         // image boundaries among them
    const long long row_step = (long long)nrh * Wrow;
    const long long img_step = (long long)Hrows * Wrow - (long long)(OH - 1) * row_step;
    const long long extra = img_step > row_step ? img_step - row_step : 0;
    const long long delta = dR * row_step + dI * extra + (OW - 1);
    return 3 + delta + max_tap + 1 + 3;
}

// pad + quantise + stream generation + OR-n accumulation with the scratch at d_workspace (capi.cu)
// w_seed_pos / w_seed_neg: see ConvPlan (13, 13 reproduces the extension)
int conv_forward(const rexsc_sc_conv_desc *desc, const void *d_act, const void *d_weight, int16_t *d_out_pos,
                 int16_t *d_out_neg, void *d_workspace, size_t workspace_bytes, cudaStream_t st, int w_seed_pos = 13,
                 int w_seed_neg = 13);

int launch_mma_probe(int blocks, int iters, int n_cols, uint32_t *d_sink, cudaStream_t st);
bool conv_tc_supported(const ConvPlan &p);
size_t conv_tc_workspace_bytes(const ConvPlan &p);
// weights -> Wb bit planes of the tensor-core kernel (sc_stream.cu)
int launch_build_lut_pair(int l, int bit_length, int gen_config, int xnor, int tw, int lw, int lwait, uint32_t *d_lut_a,
                          uint32_t *d_lut_w, cudaStream_t st);
int launch_expand_weight_bits(const ConvPlan &p, const rexsc_sc_conv_desc &d, const void *d_w, const uint32_t *d_lut,
                              uint32_t *d_Wb, cudaStream_t st);
size_t conv_tc_weight_offset(const ConvPlan &p);
// stream tables + weight bit planes + activation bit planes + status clear in one launch (sc_stream.cu);
// REXSC_E_UNSUPPORTED when the shape does not qualify and the separate launches have to be used
// opt.verify_border: check that every border pixel of the padded activation quantises to zero and set d_status[1]
//   otherwise (the caller clears the status block before the launch; the kernel then leaves it alone);
// opt.gate: run only if d_status[1] != 0 (the fallback launch after a failed verification);
// opt.skip_weights: activations only.
struct ExpandAllOptions { bool verify_border, gate, skip_weights; };
int launch_expand_all_bits(const ConvPlan &p, const rexsc_sc_conv_desc &d, const void *d_act, const void *d_w, int xnor,
                           uint32_t *d_Ab, uint32_t *d_Wb, int *d_status, const ExpandAllOptions &opt, cudaStream_t st);
// gate: 0 = run always; +1 = run only if d_status[1] == 0 (compact planes valid); -1 = only if d_status[1] != 0.
// weight_offset: byte offset of the weight bit planes in d_tc_ws (that of the standard plan, whatever grid p has).
int launch_conv_tc(const ConvPlan &p, const rexsc_sc_conv_desc &d, void *d_tc_ws, size_t weight_offset, int16_t *d_pos,
                   int16_t *d_neg, int *d_status, int gate, cudaStream_t st);

// ---- device helpers -----------------------------------------------------------------------
template <typename T> __device__ __forceinline__ float load_as_float(const T *p, long long i);
template <> __device__ __forceinline__ float load_as_float<float>(const float *p, long long i) { return p[i]; }
template <> __device__ __forceinline__ float load_as_float<__half>(const __half *p, long long i)
{
    return __half2float(p[i]);
}
template <> __device__ __forceinline__ float load_as_float<__nv_bfloat16>(const __nv_bfloat16 *p, long long i)
{
    return __bfloat162float(p[i]);
}

// ceil(clamp(x * scale, 0, scale - 1)); exact in fp32 because scale is a power of two.
__device__ __forceinline__ int quant_ceil_unipolar(float x, float scale)
{
    float v = x * scale;
    v = fminf(fmaxf(v, 0.f), scale - 1.f);
    return (int)ceilf(v);
}

} // namespace rexsc
