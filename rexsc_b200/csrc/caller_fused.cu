// Arithmetic the front end runs on the SC conv's int16 counts right after the op, as single HBM-streaming passes:
//
//   counts -> values   result.to(dtype) / bit_length for both signs and their difference
//                      (utils_functional.py:1181-1182, 1273-1274, 1316-1324: two casts, two divisions and a
//                      subtraction, five full-tensor passes in eager PyTorch)
//   calibration bins   count, sum and sum of squares of err = counts / L - guide over the 30 overlapping windows
//                      [e_i, e_i + 0.1) of the guide value, e = linspace(0, max(counts) / L, 30)
//                      (compute_bias_std_coef, utils_functional.py:901-925: 30 masked gathers, each followed by a
//                      mean and a std reduction and a host synchronisation)
//
// Both are bound by HBM: 4 B of counts in and 4-12 B of values out per element for the first, 4 B of counts
// (twice: once for the maximum, once for the bins) and the guide values for the second.
#include "common.cuh"

namespace rexsc {

namespace {

constexpr int kThreads = 256;
constexpr int kBins = 30;           // np.linspace(0, max, 30) in the reference
constexpr int kStatWarps = 4;       // warps per CTA of the bin kernel (each owns a private table)
constexpr long long kGridCap = 148LL * 8 * 2;

__device__ __forceinline__ void unpack8(const uint4 &v, int (&c)[8])
{
    const uint32_t w[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int k = 0; k < 4; k++) {
        c[2 * k] = (int)(int16_t)(w[k] & 0xffffu);
        c[2 * k + 1] = (int)(int16_t)(w[k] >> 16);
    }
}

// count -> float exactly as `.to(dtype)` gives it: fp16 rounds counts above 2048 to even, fp32 is exact
template <bool HALF> __device__ __forceinline__ float count_as(int c)
{
    return HALF ? __half2float(__int2half_rn(c)) : (float)c;
}

template <typename OUT> __device__ __forceinline__ void store8(OUT *p, long long i, const float (&v)[8]);
template <> __device__ __forceinline__ void store8<float>(float *p, long long i, const float (&v)[8])
{
    __stcs(reinterpret_cast<float4 *>(p + i), make_float4(v[0], v[1], v[2], v[3]));
    __stcs(reinterpret_cast<float4 *>(p + i) + 1, make_float4(v[4], v[5], v[6], v[7]));
}
template <> __device__ __forceinline__ void store8<__half>(__half *p, long long i, const float (&v)[8])
{
    uint4 t;
    *reinterpret_cast<__half2 *>(&t.x) = __floats2half2_rn(v[0], v[1]);
    *reinterpret_cast<__half2 *>(&t.y) = __floats2half2_rn(v[2], v[3]);
    *reinterpret_cast<__half2 *>(&t.z) = __floats2half2_rn(v[4], v[5]);
    *reinterpret_cast<__half2 *>(&t.w) = __floats2half2_rn(v[6], v[7]);
    __stcs(reinterpret_cast<uint4 *>(p + i), t);
}
template <typename OUT> __device__ __forceinline__ OUT to_out(float v);
template <> __device__ __forceinline__ float to_out<float>(float v) { return v; }
template <> __device__ __forceinline__ __half to_out<__half>(float v) { return __float2half_rn(v); }
template <typename OUT> __device__ __forceinline__ float round_out(float v);
template <> __device__ __forceinline__ float round_out<float>(float v) { return v; }
template <> __device__ __forceinline__ float round_out<__half>(float v) { return __half2float(__float2half_rn(v)); }

// ---- counts -> values --------------------------------------------------------------------------------------
// Eight elements per thread per iteration: one 128-bit load per sign, 128-bit stores.  `inv_l` is a power of two,
// so every product is exact and the only roundings are the ones the eager sequence has (count -> fp16 above 2048,
// the fp16 difference).
template <typename OUT>
__global__ void __launch_bounds__(kThreads)
counts_to_value_kernel(const int16_t *__restrict__ pos, const int16_t *__restrict__ neg, OUT *__restrict__ vpos,
                       OUT *__restrict__ vneg, OUT *__restrict__ vdiff, long long n, float inv_l, int vec_ok)
{
    constexpr bool HALF = sizeof(OUT) == 2;
    const long long n_groups = (n + 7) >> 3;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n_groups; g += stride) {
        const long long i = g << 3;
        const int valid = (int)(n - i < 8 ? n - i : 8);
        int cp[8], cn[8];
        if (vec_ok && valid == 8) {
            unpack8(__ldcs(reinterpret_cast<const uint4 *>(pos + i)), cp);
            unpack8(__ldcs(reinterpret_cast<const uint4 *>(neg + i)), cn);
        } else {
#pragma unroll
            for (int k = 0; k < 8; k++) {
                cp[k] = k < valid ? pos[i + k] : 0;
                cn[k] = k < valid ? neg[i + k] : 0;
            }
        }
        float a[8], b[8], d[8];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            a[k] = round_out<OUT>(count_as<HALF>(cp[k]) * inv_l);
            b[k] = round_out<OUT>(count_as<HALF>(cn[k]) * inv_l);
            d[k] = a[k] - b[k];
        }
        if (vec_ok && valid == 8) {
            if (vpos) store8<OUT>(vpos, i, a);
            if (vneg) store8<OUT>(vneg, i, b);
            if (vdiff) store8<OUT>(vdiff, i, d);
        } else {
#pragma unroll
            for (int k = 0; k < 8; k++)
                if (k < valid) {
                    if (vpos) vpos[i + k] = to_out<OUT>(a[k]);
                    if (vneg) vneg[i + k] = to_out<OUT>(b[k]);
                    if (vdiff) vdiff[i + k] = to_out<OUT>(d[k]);
                }
        }
    }
}

// eight guide values as loaded (registers of a prefetched group) and as floats
template <typename G> struct Guide8;
template <> struct Guide8<float> {
    float4 a, b;
    __device__ __forceinline__ void load(const float *p, long long i)
    {
        a = __ldcs(reinterpret_cast<const float4 *>(p + i));
        b = __ldcs(reinterpret_cast<const float4 *>(p + i) + 1);
    }
    __device__ __forceinline__ void unpack(float *v) const
    {
        v[0] = a.x; v[1] = a.y; v[2] = a.z; v[3] = a.w;
        v[4] = b.x; v[5] = b.y; v[6] = b.z; v[7] = b.w;
    }
};
template <> struct Guide8<__half> {
    uint4 t;
    __device__ __forceinline__ void load(const __half *p, long long i)
    {
        t = __ldcs(reinterpret_cast<const uint4 *>(p + i));
    }
    __device__ __forceinline__ void unpack(float *v) const
    {
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
            v[2 * k] = f.x;
            v[2 * k + 1] = f.y;
        }
    }
};

// ---- calibration bins ----------------------------------------------------------------------------------------
// Result block in device memory (REXSC_CALIB_STATS_BYTES):
//   double sums[30][3]   per window: number of elements, sum of err, sum of err^2
//   int32  max_count     largest count of either sign
//   int32  reserved
struct CalibStats {
    double sums[kBins][3];
    int max_count;
    int reserved;
};
static_assert(sizeof(CalibStats) == REXSC_CALIB_STATS_BYTES, "result block size is part of the C ABI");

__global__ void __launch_bounds__(kThreads)
max_count_kernel(const int16_t *__restrict__ pos, const int16_t *__restrict__ neg, long long n, int vec_ok,
                 CalibStats *__restrict__ out)
{
    int m = 0;
    const long long n_groups = (n + 7) >> 3;
    const long long n_full = n >> 3; // groups that hold eight elements
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec_ok) {
        // four groups (eight 128-bit loads) in flight per thread
        for (; g + 3 * stride < n_full; g += 4 * stride) {
            uint4 v[8];
#pragma unroll
            for (int u = 0; u < 4; u++) {
                v[2 * u] = __ldcs(reinterpret_cast<const uint4 *>(pos + ((g + u * stride) << 3)));
                v[2 * u + 1] = __ldcs(reinterpret_cast<const uint4 *>(neg + ((g + u * stride) << 3)));
            }
#pragma unroll
            for (int u = 0; u < 8; u++) {
                // packed signed 16-bit maxima, two counts per instruction
                const uint32_t w[4] = {v[u].x, v[u].y, v[u].z, v[u].w};
                uint32_t t = __vmaxs2(__vmaxs2(w[0], w[1]), __vmaxs2(w[2], w[3]));
                m = max(m, max((int)(int16_t)(t & 0xffffu), (int)(int16_t)(t >> 16)));
            }
        }
    }
    for (; g < n_groups; g += stride) {
        const long long i = g << 3;
        const int valid = (int)(n - i < 8 ? n - i : 8);
        if (vec_ok && valid == 8) {
            int cp[8], cn[8];
            unpack8(__ldcs(reinterpret_cast<const uint4 *>(pos + i)), cp);
            unpack8(__ldcs(reinterpret_cast<const uint4 *>(neg + i)), cn);
#pragma unroll
            for (int k = 0; k < 8; k++) m = max(m, max(cp[k], cn[k]));
        } else {
            for (int k = 0; k < valid; k++) m = max(m, max((int)pos[i + k], (int)neg[i + k]));
        }
    }
    m = __reduce_max_sync(0xffffffffu, m);
    if ((threadIdx.x & 31) == 0 && m > 0) atomicMax(&out->max_count, m);
}

// Window edges exactly as the reference's host code makes them: numpy's linspace in float64 (i * (max / 29), the
// last one set to max), `start + 0.1` in float64, and the comparison against an fp32 tensor with the scalar
// converted to fp32.
__device__ __forceinline__ void window_edges(int i, double top, float &lo, float &hi)
{
    const double step = top / (double)(kBins - 1);
    const double e = i == kBins - 1 ? top : __dmul_rn((double)i, step);
    lo = (float)e;
    hi = (float)__dadd_rn(e, 0.1);
}

// The 30 start edges and the 30 end edges cut the axis into 61 cells; an element with `cl` start edges and `ch`
// end edges at or below its guide value lies in the windows ch <= b < cl and in cell cl + ch.  The kernel adds
// every element to exactly one cell and turns cells into windows once per CTA at the end.
constexpr int kCells = 2 * kBins + 1;
constexpr int kBuckets = 512;

template <typename G, bool HALF>
__global__ void __launch_bounds__(kStatWarps * 32)
calib_bins_kernel(const int16_t *__restrict__ pos, const int16_t *__restrict__ neg, const G *__restrict__ gpos,
                  const G *__restrict__ gneg, long long n, float inv_l, int vec_ok, int gvec_ok,
                  CalibStats *__restrict__ out)
{
    // One private table per warp, one column per lane: tab[warp][cell][which][lane].  A lane only ever touches its
    // own column (bank = lane), so the read-modify-writes need neither atomics nor conflict resolution.
    extern __shared__ __align__(16) unsigned char smem_raw[];
    float(*tab)[kCells][3][32] = reinterpret_cast<float(*)[kCells][3][32]>(smem_raw);
    // edge tables with one sentinel on each side: e_lo[j + 1] = start of window j, e_lo[0] = -inf, e_lo[31] = NaN
    __shared__ float e_lo[kBins + 2], e_hi[kBins + 2];
    __shared__ int cell_cl[kCells], cell_ch[kCells];
    __shared__ double cell_sum[kCells][3];
    const int warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (int k = threadIdx.x; k < kStatWarps * kCells * 3 * 32; k += blockDim.x) (&tab[0][0][0][0])[k] = 0.f;
    const double top = (double)count_as<HALF>(out->max_count) * (double)inv_l;
    if (threadIdx.x < kBins) window_edges(threadIdx.x, top, e_lo[threadIdx.x + 1], e_hi[threadIdx.x + 1]);
    if (threadIdx.x == 0) {
        e_lo[0] = e_hi[0] = -INFINITY;
        e_lo[kBins + 1] = e_hi[kBins + 1] = NAN; // NaN <= x is false for every x
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        // walk the merged edge list: cell c lies after c edges, i of them starts and j ends
        int i = 0, j = 0;
        for (int c = 0; c < kCells; c++) {
            cell_cl[c] = i;
            cell_ch[c] = j;
            if (i < kBins && (j >= kBins || e_lo[i + 1] <= e_hi[j + 1])) i++;
            else j++;
        }
    }
    const float step = (float)(top / (double)(kBins - 1));
    const bool flat = !(step > 0.f);             // every count is zero: all windows are [0, 0.1)
    const float inv_step = flat ? 0.f : 1.f / step;
    const float lo0 = e_lo[1], hi0 = e_hi[1];

    // Bucket table: the axis from 0 to beyond the last window end in buckets half a window spacing wide.  A bucket
    // stores how many of the 60 edges lie a quarter bucket or more below it (x = base) and the at most two edges
    // (one start, one end: same-kind edges are a full spacing apart) from there to a quarter bucket above it
    // (y, z; NaN if absent), so an element's cell is base + (y <= x) + (z <= x): one 128-bit load and two exact
    // comparisons.  The quarter-bucket overlap absorbs the rounding of the bucket index.  Used when the table fits
    // (maximum count / L of about 0.02 and more); otherwise the per-table estimates below decide.
    __shared__ float4 bucket[kBuckets];
    const float bw = 0.5f * step;
    const float inv_bw = flat ? 0.f : 1.f / bw;
    const float n_need = flat ? 0.f : ((float)top + 0.1f) * inv_bw + 3.f;
    const bool use_buckets = !flat && n_need < (float)kBuckets;
    const int n_buckets = use_buckets ? (int)n_need : 0;
    for (int t = threadIdx.x; t < n_buckets; t += blockDim.x) {
        const float lower = ((float)t - 0.25f) * bw, upper = ((float)t + 1.25f) * bw;
        int base = 0;
        float y = NAN, z = NAN;
        // starts and ends are each ascending, so the first edge of a kind above `lower` is the only candidate of it
        float cs = NAN, ce = NAN;
        for (int j = kBins; j >= 1; j--) {
            if (e_lo[j] <= lower) base++; else cs = e_lo[j];
            if (e_hi[j] <= lower) base++; else ce = e_hi[j];
        }
        if (!(cs <= upper)) cs = NAN;
        if (!(ce <= upper)) ce = NAN;
        y = cs; z = ce;
        bucket[t] = make_float4(__int_as_float(base), y, z, 0.f);
    }
    __syncthreads();

    // Number T of edges of a sentinel-padded table that are <= x.  q estimates x / spacing with an error far below
    // one (stream lengths up to 4096), so floor(q) is T - 1 give or take one: edges below index floor(q) are <= x
    // for certain, edges from floor(q) + 2 on are above it, and two exact comparisons decide the rest.  NaN and
    // negative x give 0.
    auto edges_below = [&](const float *tbl, float q, float x) -> int {
        const int cand = q >= (float)(kBins - 1) ? kBins - 1 : (q > 0.f ? (int)q : 0);
        return cand + (tbl[cand + 1] <= x) + (tbl[cand + 2] <= x);
    };
    auto cell_of = [&](float x) -> int {
        if (flat) return (x >= lo0 ? kBins : 0) + (x >= hi0 ? kBins : 0);
        if (use_buckets) {
            const float q = fminf(fmaxf(x * inv_bw, 0.f), (float)(n_buckets - 1)); // NaN -> bucket 0, cell 0
            const float4 b = bucket[(int)q];
            return __float_as_int(b.x) + (b.y <= x) + (b.z <= x);
        }
        return edges_below(e_lo, x * inv_step, x) + edges_below(e_hi, (x - 0.1f) * inv_step, x);
    };

    float(*mine)[3][32] = tab[warp];
    // sixteen elements (eight of each sign) into the warp's table
    auto accumulate = [&](const int (&cp)[8], const int (&cn)[8], const float (&x)[16]) {
        int cell[16];
#pragma unroll
        for (int k = 0; k < 16; k++) cell[k] = cell_of(x[k]);
        // Table updates four elements at a time: the four columns are loaded together (one shared-memory round trip
        // instead of four dependent ones); an element whose cell equals an earlier one of the group continues from
        // that element's updated values in registers, and the stores go out in order so the last one stands.
#pragma unroll
        for (int k0 = 0; k0 < 16; k0 += 4) {
            float *col[4];
            float c[4], s1[4], s2[4], err[4];
#pragma unroll
            for (int j = 0; j < 4; j++) {
                const int k = k0 + j;
                err[j] = count_as<HALF>(k < 8 ? cp[k] : cn[k - 8]) * inv_l - x[k];
                col[j] = &mine[cell[k]][0][lane];
                c[j] = col[j][0];
                s1[j] = col[j][32];
                s2[j] = col[j][64];
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
#pragma unroll
                for (int i = 0; i < j; i++) {   // later i overrides earlier: it already carries their sums
                    const bool same = cell[k0 + i] == cell[k0 + j];
                    c[j] = same ? c[i] : c[j];
                    s1[j] = same ? s1[i] : s1[j];
                    s2[j] = same ? s2[i] : s2[j];
                }
                c[j] += 1.f;
                s1[j] += err[j];
                s2[j] = fmaf(err[j], err[j], s2[j]);
            }
#pragma unroll
            for (int j = 0; j < 4; j++) {
                col[j][0] = c[j];
                col[j][32] = s1[j];
                col[j][64] = s2[j];
            }
        }
    };

    const long long n_groups = (n + 7) >> 3;
    const long long n_full = n >> 3;
    const long long stride = (long long)gridDim.x * blockDim.x;
    long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x;
    if (vec_ok && gvec_ok) {
        // whole groups through 128-bit loads, the next group's loads in flight while this one is processed (two
        // warps per scheduler do not hide a DRAM round trip by themselves)
        uint4 rp, rn;
        Guide8<G> qp, qn;
        if (g < n_full) {
            rp = __ldcs(reinterpret_cast<const uint4 *>(pos + (g << 3)));
            rn = __ldcs(reinterpret_cast<const uint4 *>(neg + (g << 3)));
            qp.load(gpos, g << 3);
            qn.load(gneg, g << 3);
        }
        for (; g < n_full; g += stride) {
            const uint4 cur_p = rp, cur_n = rn;
            const Guide8<G> cur_qp = qp, cur_qn = qn;
            const long long nxt = g + stride;
            if (nxt < n_full) {
                rp = __ldcs(reinterpret_cast<const uint4 *>(pos + (nxt << 3)));
                rn = __ldcs(reinterpret_cast<const uint4 *>(neg + (nxt << 3)));
                qp.load(gpos, nxt << 3);
                qn.load(gneg, nxt << 3);
            }
            int cp[8], cn[8];
            float x[16];
            unpack8(cur_p, cp);
            unpack8(cur_n, cn);
            cur_qp.unpack(&x[0]);
            cur_qn.unpack(&x[8]);
            accumulate(cp, cn, x);
        }
    }
    // unaligned inputs and the ragged last group: element-wise loads
    for (; g < n_groups; g += stride) {
        const long long i = g << 3;
        const int valid = (int)(n - i < 8 ? n - i : 8);
        int cp[8], cn[8];
        float x[16];
#pragma unroll
        for (int k = 0; k < 8; k++) {
            cp[k] = k < valid ? pos[i + k] : 0;
            cn[k] = k < valid ? neg[i + k] : 0;
            // padding gets a guide value of NaN, which lands in cell 0; that cell belongs to no window
            x[k] = k < valid ? load_as_float<G>(gpos, i + k) : NAN;
            x[8 + k] = k < valid ? load_as_float<G>(gneg, i + k) : NAN;
        }
        accumulate(cp, cn, x);
    }
    __syncthreads();
    // cells: every warp folds its share of the 183 entries over the 4 tables and the 32 columns, in double
    for (int e = warp; e < kCells * 3; e += kStatWarps) {
        double s = 0.0;
#pragma unroll
        for (int w = 0; w < kStatWarps; w++) s += (double)tab[w][e / 3][e % 3][lane];
#pragma unroll
        for (int d = 16; d > 0; d >>= 1) s += __shfl_xor_sync(0xffffffffu, s, d);
        if (lane == 0) cell_sum[e / 3][e % 3] = s;
    }
    __syncthreads();
    // windows from cells, one atomic per CTA per entry.  Cell 0 (below every window) also collects the NaN
    // padding of a ragged tail; it is part of no window.
    for (int e = threadIdx.x; e < kBins * 3; e += blockDim.x) {
        const int b = e / 3, k = e % 3;
        double s = 0.0;
        for (int c = 1; c < kCells; c++)
            if (cell_ch[c] <= b && b < cell_cl[c]) s += cell_sum[c][k];
        if (s != 0.0) atomicAdd(&out->sums[b][k], s);
    }
}

constexpr size_t kStatSmem = (size_t)kStatWarps * kCells * 3 * 32 * sizeof(float);

inline bool aligned16(const void *p) { return (reinterpret_cast<uintptr_t>(p) & 15) == 0; }
inline bool pow2(int v) { return v > 0 && (v & (v - 1)) == 0; }
inline unsigned grid_for(long long n, int threads)
{
    long long blocks = ((n + 7) / 8 + threads - 1) / threads;
    if (blocks > kGridCap) blocks = kGridCap;
    return (unsigned)(blocks < 1 ? 1 : blocks);
}

} // namespace

} // namespace rexsc

using namespace rexsc;

extern "C" int rexsc_sc_counts_to_value(const int16_t *d_pos, const int16_t *d_neg, int32_t bit_length,
                                        int32_t out_dtype, void *d_val_pos, void *d_val_neg, void *d_val_diff,
                                        int64_t n_elem, void *stream)
{
    if (n_elem < 0 || (!d_val_pos && !d_val_neg && !d_val_diff)) return REXSC_E_BAD_ARG;
    if (!pow2(bit_length)) return REXSC_E_UNSUPPORTED; // the scaling is exact only for power-of-two stream lengths
    if (out_dtype != REXSC_F32 && out_dtype != REXSC_F16) return REXSC_E_UNSUPPORTED;
    if (n_elem == 0) return REXSC_OK;
    if (!d_pos || !d_neg) return REXSC_E_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    const int vec = aligned16(d_pos) && aligned16(d_neg) && aligned16(d_val_pos) && aligned16(d_val_neg) &&
                    aligned16(d_val_diff);
    const float inv_l = 1.f / (float)bit_length;
    const unsigned grid = grid_for(n_elem, kThreads);
    if (out_dtype == REXSC_F32)
        counts_to_value_kernel<float><<<grid, kThreads, 0, st>>>(d_pos, d_neg, (float *)d_val_pos, (float *)d_val_neg,
                                                                 (float *)d_val_diff, n_elem, inv_l, vec);
    else
        counts_to_value_kernel<__half><<<grid, kThreads, 0, st>>>(d_pos, d_neg, (__half *)d_val_pos,
                                                                  (__half *)d_val_neg, (__half *)d_val_diff, n_elem,
                                                                  inv_l, vec);
    REXSC_LAUNCH_CHECK("counts_to_value_kernel");
    return REXSC_OK;
}

static int calib_check(const int16_t *d_pos, const int16_t *d_neg, const void *d_guide_pos, const void *d_guide_neg,
                       bool need_guides, int32_t guide_dtype, int32_t bit_length, int64_t n_elem, void *d_stats)
{
    if (n_elem < 0 || !d_stats || (reinterpret_cast<uintptr_t>(d_stats) & 7)) return REXSC_E_BAD_ARG;
    // up to 4096 the fp32 estimate of an element's window is within one of the exact answer (the kernel relies on it)
    if (!pow2(bit_length) || bit_length > 4096) return REXSC_E_UNSUPPORTED;
    if (n_elem > 0 && (!d_pos || !d_neg)) return REXSC_E_BAD_ARG;
    if (need_guides) {
        if (n_elem > 0 && (!d_guide_pos || !d_guide_neg)) return REXSC_E_BAD_ARG;
        if (guide_dtype != REXSC_F32 && guide_dtype != REXSC_F16) return REXSC_E_UNSUPPORTED;
    }
    return REXSC_OK;
}

extern "C" int rexsc_sc_calib_max(const int16_t *d_pos, const int16_t *d_neg, int32_t bit_length, int64_t n_elem,
                                  void *d_stats, void *stream)
{
    const int rc = calib_check(d_pos, d_neg, nullptr, nullptr, false, 0, bit_length, n_elem, d_stats);
    if (rc != REXSC_OK) return rc;
    cudaStream_t st = (cudaStream_t)stream;
    CalibStats *out = (CalibStats *)d_stats;
    REXSC_CUDA_CHECK(cudaMemsetAsync(out, 0, sizeof(CalibStats), st));
    if (n_elem == 0) return REXSC_OK;
    const int vec = aligned16(d_pos) && aligned16(d_neg);
    // at least four groups per thread where the input allows, so that the unrolled loop of the kernel runs
    unsigned max_grid = grid_for((n_elem + 3) / 4, kThreads);
    if (max_grid > 148u * 8u) max_grid = 148u * 8u;
    max_count_kernel<<<max_grid, kThreads, 0, st>>>(d_pos, d_neg, n_elem, vec, out);
    REXSC_LAUNCH_CHECK("max_count_kernel");
    return REXSC_OK;
}

extern "C" int rexsc_sc_calib_windows(const int16_t *d_pos, const int16_t *d_neg, const void *d_guide_pos,
                                      const void *d_guide_neg, int32_t guide_dtype, int32_t bit_length,
                                      int32_t counts_via_half, int64_t n_elem, void *d_stats, void *stream)
{
    const int rc = calib_check(d_pos, d_neg, d_guide_pos, d_guide_neg, true, guide_dtype, bit_length, n_elem, d_stats);
    if (rc != REXSC_OK) return rc;
    if (n_elem == 0) return REXSC_OK;
    cudaStream_t st = (cudaStream_t)stream;
    CalibStats *out = (CalibStats *)d_stats;
    const int vec = aligned16(d_pos) && aligned16(d_neg);
    const int gvec = aligned16(d_guide_pos) && aligned16(d_guide_neg);
    const float inv_l = 1.f / (float)bit_length;
    // two CTAs fit an SM (94 KB of tables each): one persistent wave, one fold per CTA
    unsigned grid = grid_for(n_elem, kStatWarps * 32);
    if (grid > 148u * 2u) grid = 148u * 2u;
#define REXSC_CALIB_LAUNCH(G, H)                                                                                  \
    do {                                                                                                          \
        REXSC_CUDA_CHECK(cudaFuncSetAttribute(calib_bins_kernel<G, H>, cudaFuncAttributeMaxDynamicSharedMemorySize, \
                                              (int)kStatSmem));                                                   \
        calib_bins_kernel<G, H><<<grid, kStatWarps * 32, kStatSmem, st>>>(                                        \
            d_pos, d_neg, (const G *)d_guide_pos, (const G *)d_guide_neg, n_elem, inv_l, vec, gvec, out);         \
    } while (0)
    if (guide_dtype == REXSC_F32) {
        if (counts_via_half) REXSC_CALIB_LAUNCH(float, true);
        else REXSC_CALIB_LAUNCH(float, false);
    } else {
        if (counts_via_half) REXSC_CALIB_LAUNCH(__half, true);
        else REXSC_CALIB_LAUNCH(__half, false);
    }
#undef REXSC_CALIB_LAUNCH
    REXSC_LAUNCH_CHECK("calib_bins_kernel");
    return REXSC_OK;
}

extern "C" int rexsc_sc_calib_stats(const int16_t *d_pos, const int16_t *d_neg, const void *d_guide_pos,
                                    const void *d_guide_neg, int32_t guide_dtype, int32_t bit_length,
                                    int32_t counts_via_half, int64_t n_elem, void *d_stats, void *stream)
{
    int rc = calib_check(d_pos, d_neg, d_guide_pos, d_guide_neg, true, guide_dtype, bit_length, n_elem, d_stats);
    if (rc != REXSC_OK) return rc;
    rc = rexsc_sc_calib_max(d_pos, d_neg, bit_length, n_elem, d_stats, stream);
    if (rc != REXSC_OK) return rc;
    return rexsc_sc_calib_windows(d_pos, d_neg, d_guide_pos, d_guide_neg, guide_dtype, bit_length, counts_via_half,
                                  n_elem, d_stats, stream);
}
