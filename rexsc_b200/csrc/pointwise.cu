// Point-wise OR-n activation, calibration (bias polynomial) and error injection (std polynomial x N(0,1))
// as 128-bit vectorised HBM-streaming kernels.
//
// Math (torch_c/sc-extension/sc_device.cuh:393-430 forward, :466-505 derivative, :507-545 polynomials):
//   f_n(s)  = n - e^{-s} * sum_{i<n} (n-i) s^i / i!        evaluated as a chain of fmaf(-(c_i s^i), e, x)
//   f_n'(s) = e^{-s} * sum_{i<n} s^i / i!
//   y(x, eps) = x + B(x) + S(x) * eps,  B, S 5th-order polynomials (Horner-free: powers then fmaf, as the
//   reference evaluates them), dy/dx = 1 + B'(x) with the noise held constant.
// The fp32 operation order follows the reference's so that results agree to the last bit wherever the same
// hardware exp approximation (__expf) is used; only the random stream differs (counter-based Philox here,
// persistent cuRAND states there: sc_cuda_pw.cu:699-706).
#include "common.cuh"

namespace rexsc {

namespace {

constexpr int kPwThreads = 256;

// ---- scalar math --------------------------------------------------------------------------------
template <int N> __device__ __forceinline__ float orn_forward(float s)
{
    const float e = __expf(-s);
    if (N == 1) return 1.f - e;
    float x = fmaf(-(float)N, e, (float)N);
    if (N == 2) return fmaf(-s, e, x);
    const float s2 = s * s;
    if (N == 3) {
        x = fmaf(-2.f * s, e, x);
        return fmaf(-0.5f * s2, e, x);
    }
    x = fmaf(-3.f * s, e, x);
    const float s3 = s2 * s;
    x = fmaf(-s2, e, x);
    return fmaf((-1.f / 6.f) * s3, e, x);
}

// e^{-s} * sum_{i<n} s^i / i!, given e = __expf(-s)
template <int N> __device__ __forceinline__ float orn_derivative(float s, float e)
{
    if (N == 1) return e;
    float d = fmaf(s, e, e);
    if (N == 2) return d;
    const float s2 = s * s;
    if (N == 3) return fmaf(0.5f * s2, e, d);
    const float s3 = s2 * s;
    d = fmaf(0.5f * s2, e, d);
    return fmaf((1.f / 6.f) * s3, e, d);
}

struct Coef6 { float c[6]; };

__device__ __forceinline__ Coef6 load_coef(const float *p)
{
    Coef6 r;
#pragma unroll
    for (int i = 0; i < 6; i++) r.c[i] = __ldg(p + i);
    return r;
}

// mean part x + B(x) and noise scale S(x) of the injection model, evaluated with shared powers
__device__ __forceinline__ void inject_terms(float x, const Coef6 &b, const Coef6 &sd, float &mean, float &scale)
{
    const float x2 = x * x;
    float xb = fmaf(b.c[1], x, b.c[0]);
    const float x3 = x2 * x;
    xb = fmaf(b.c[2], x2, xb);
    const float x4 = x3 * x;
    xb = fmaf(b.c[3], x3, xb);
    const float x5 = x4 * x;
    xb = fmaf(b.c[4], x4, xb);
    xb = fmaf(b.c[5], x5, xb);
    float xs = fmaf(sd.c[1], x, sd.c[0]);
    xs = fmaf(sd.c[2], x2, xs);
    xs = fmaf(sd.c[3], x3, xs);
    xs = fmaf(sd.c[4], x4, xs);
    xs = fmaf(sd.c[5], x5, xs);
    mean = x + xb;
    scale = xs;
}

__device__ __forceinline__ float inject(float x, float eps, const Coef6 &b, const Coef6 &sd)
{
    const float x2 = x * x;
    float xb = fmaf(b.c[1], x, b.c[0]);
    const float x3 = x2 * x;
    xb = fmaf(b.c[2], x2, xb);
    const float x4 = x3 * x;
    xb = fmaf(b.c[3], x3, xb);
    const float x5 = x4 * x;
    xb = fmaf(b.c[4], x4, xb);
    xb = fmaf(b.c[5], x5, xb);
    float xs = fmaf(sd.c[1], x, sd.c[0]);
    xs = fmaf(sd.c[2], x2, xs);
    xs = fmaf(sd.c[3], x3, xs);
    xs = fmaf(sd.c[4], x4, xs);
    xs = fmaf(sd.c[5], x5, xs);
    return x + xb + xs * eps;
}

__device__ __forceinline__ float inject_derivative(float x, const Coef6 &b)
{
    const float x2 = x * x;
    float d = fmaf(2.f * b.c[2], x, 1.f + b.c[1]);
    const float x3 = x2 * x;
    d = fmaf(3.f * b.c[3], x2, d);
    d = fmaf(4.f * b.c[4], x3, d);
    const float x4 = x3 * x;
    return fmaf(5.f * b.c[5], x4, d);
}

// backward through y(f_n(s)): g * (1 + B'(f_n(s))) * f_n'(s)
template <int N> __device__ __forceinline__ float orn_inject_backward(float g, float s, const Coef6 &b)
{
    const float e = __expf(-s);
    float x;
    if (N == 1) x = 1.f - e;
    else {
        x = fmaf(-(float)N, e, (float)N);
        if (N == 2) x = fmaf(-s, e, x);
        else if (N == 3) { x = fmaf(-2.f * s, e, x); x = fmaf(-0.5f * (s * s), e, x); }
        else {
            const float s2 = s * s;
            x = fmaf(-3.f * s, e, x);
            const float s3 = s2 * s;
            x = fmaf(-s2, e, x);
            x = fmaf((-1.f / 6.f) * s3, e, x);
        }
    }
    float xd = inject_derivative(x, b) * g;
    return orn_derivative<N>(s, e) * xd;
}

__device__ __forceinline__ float round_to_half(float v) { return __half2float(__float2half_rn(v)); }

// ---- Philox4x32-10 (Salmon et al., SC'11) + Box-Muller -------------------------------------------
__device__ __forceinline__ uint4 philox4x32_10(uint4 ctr, uint2 key)
{
#pragma unroll
    for (int r = 0; r < 10; r++) {
        const uint32_t hi0 = __umulhi(0xD2511F53u, ctr.x), lo0 = 0xD2511F53u * ctr.x;
        const uint32_t hi1 = __umulhi(0xCD9E8D57u, ctr.z), lo1 = 0xCD9E8D57u * ctr.z;
        ctr = make_uint4(hi1 ^ ctr.y ^ key.x, lo1, hi0 ^ ctr.w ^ key.y, lo0);
        key.x += 0x9E3779B9u;
        key.y += 0xBB67AE85u;
    }
    return ctr;
}

__device__ __forceinline__ void box_muller(uint32_t a, uint32_t b, float &n0, float &n1)
{
    const float u = fmaf((float)a, 2.3283064365386963e-10f, 1.1641532182693481e-10f); // (0, 1]
    const float v = fmaf((float)b, 2.3283064365386963e-10f, 1.1641532182693481e-10f);
    const float r = sqrtf(-2.f * __logf(u));
    float sn, cs;
    __sincosf(6.2831853071795865f * v, &sn, &cs);
    n0 = r * sn;
    n1 = r * cs;
}

// four standard normals for element group `grp` (4 consecutive elements), stream `which`
__device__ __forceinline__ void normal4(uint64_t seed, uint64_t offset, uint64_t grp, uint32_t which, float (&z)[4])
{
    const uint4 ctr = make_uint4((uint32_t)grp, (uint32_t)(grp >> 32), (uint32_t)offset,
                                 ((uint32_t)(offset >> 32) << 1) ^ which);
    const uint4 r = philox4x32_10(ctr, make_uint2((uint32_t)seed, (uint32_t)(seed >> 32)));
    box_muller(r.x, r.y, z[0], z[1]);
    box_muller(r.z, r.w, z[2], z[3]);
}

// ---- 4-element vector access ----------------------------------------------------------------------
template <typename T> struct V4;
template <> struct V4<float> {
    static constexpr int kAlign = 16;
    static __device__ __forceinline__ void load(const float *p, long long i, float (&v)[4])
    {
        const float4 t = __ldcs(reinterpret_cast<const float4 *>(p + i));
        v[0] = t.x; v[1] = t.y; v[2] = t.z; v[3] = t.w;
    }
    static __device__ __forceinline__ void store(float *p, long long i, const float (&v)[4])
    {
        __stcs(reinterpret_cast<float4 *>(p + i), make_float4(v[0], v[1], v[2], v[3]));
    }
};
template <> struct V4<__half> {
    static constexpr int kAlign = 8;
    static __device__ __forceinline__ void load(const __half *p, long long i, float (&v)[4])
    {
        const uint2 t = __ldcs(reinterpret_cast<const uint2 *>(p + i));
        const float2 a = __half22float2(*reinterpret_cast<const __half2 *>(&t.x));
        const float2 b = __half22float2(*reinterpret_cast<const __half2 *>(&t.y));
        v[0] = a.x; v[1] = a.y; v[2] = b.x; v[3] = b.y;
    }
    static __device__ __forceinline__ void store(__half *p, long long i, const float (&v)[4])
    {
        uint2 t;
        *reinterpret_cast<__half2 *>(&t.x) = __floats2half2_rn(v[0], v[1]);
        *reinterpret_cast<__half2 *>(&t.y) = __floats2half2_rn(v[2], v[3]);
        __stcs(reinterpret_cast<uint2 *>(p + i), t);
    }
};
template <> struct V4<__nv_bfloat16> {
    static constexpr int kAlign = 8;
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, long long i, float (&v)[4])
    {
        const uint2 t = __ldcs(reinterpret_cast<const uint2 *>(p + i));
        v[0] = __uint_as_float(t.x << 16); v[1] = __uint_as_float(t.x & 0xffff0000u);
        v[2] = __uint_as_float(t.y << 16); v[3] = __uint_as_float(t.y & 0xffff0000u);
    }
};

// Streaming driver: OP::apply(group index, first element index, n valid in [1,4], vectorised?) does the work
// for 4 consecutive elements.  Grid-stride over groups, two groups in flight per thread per iteration.
template <typename OP> __global__ void __launch_bounds__(kPwThreads) pw_kernel(OP op, long long n_elem, int vec_ok)
{
    const long long n_groups = (n_elem + 3) >> 2;
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long g = (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n_groups; g += stride) {
        const long long i = g << 2;
        const int valid = (int)(n_elem - i < 4 ? n_elem - i : 4);
        op.apply(g, i, valid, vec_ok && valid == 4);
    }
}

template <typename T> __device__ __forceinline__ void load4(const T *p, long long i, int valid, bool vec, float (&v)[4])
{
    if (vec) { V4<T>::load(p, i, v); return; }
#pragma unroll
    for (int k = 0; k < 4; k++) v[k] = k < valid ? load_as_float<T>(p, i + k) : 0.f;
}
__device__ __forceinline__ void store4(float *p, long long i, int valid, bool vec, const float (&v)[4])
{
    if (vec) { V4<float>::store(p, i, v); return; }
#pragma unroll
    for (int k = 0; k < 4; k++) if (k < valid) p[i + k] = v[k];
}
__device__ __forceinline__ void store4h(__half *p, long long i, int valid, bool vec, const float (&v)[4])
{
    if (vec) { V4<__half>::store(p, i, v); return; }
#pragma unroll
    for (int k = 0; k < 4; k++) if (k < valid) p[i + k] = __float2half_rn(v[k]);
}

// ---- the six ops ----------------------------------------------------------------------------------
template <typename T, int N> struct OrnFwd {
    const T *in; float *out;
    __device__ __forceinline__ void apply(long long, long long i, int valid, bool vec) const
    {
        float v[4];
        load4<T>(in, i, valid, vec, v);
#pragma unroll
        for (int k = 0; k < 4; k++) v[k] = orn_forward<N>(v[k]);
        store4(out, i, valid, vec, v);
    }
};

template <typename T, int N> struct OrnBwd {
    const float *grad; const T *in; float *gin;
    __device__ __forceinline__ void apply(long long, long long i, int valid, bool vec) const
    {
        float s[4], g[4];
        load4<T>(in, i, valid, vec, s);
        load4<float>(grad, i, valid, vec, g);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float sh = round_to_half(s[k]); // the reference casts the saved sum to fp16 (sc_cuda_pw.cu:775)
            const float e = __expf(-sh);
            g[k] = orn_derivative<N>(sh, e) * g[k];
        }
        store4(gin, i, valid, vec, g);
    }
};

template <typename T, int N> struct BothFwd {
    const T *pos, *neg; float *out; const float *bias, *stdc; uint64_t seed, offset;
    __device__ __forceinline__ void apply(long long grp, long long i, int valid, bool vec) const
    {
        const Coef6 b = load_coef(bias), sd = load_coef(stdc);
        float p[4], q[4], z[4];
        load4<T>(pos, i, valid, vec, p);
        load4<T>(neg, i, valid, vec, q);
        // The reference draws one normal per sign, S(xp)*e1 - S(xn)*e2; the difference of two independent
        // Gaussians is one Gaussian of variance S(xp)^2 + S(xn)^2, so a single draw per element gives the same
        // output distribution with half the random numbers.
        normal4(seed, offset, (uint64_t)grp, 0u, z);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            float mp, sp, mn, sn;
            inject_terms(orn_forward<N>(p[k]), b, sd, mp, sp);
            inject_terms(orn_forward<N>(q[k]), b, sd, mn, sn);
            p[k] = fmaf(sqrtf(fmaf(sp, sp, sn * sn)), z[k], mp - mn);
        }
        store4(out, i, valid, vec, p);
    }
};

template <typename T, int N> struct BothBwd {
    const float *grad; const T *pos, *neg; float *gp, *gn; const float *bias;
    __device__ __forceinline__ void apply(long long, long long i, int valid, bool vec) const
    {
        const Coef6 b = load_coef(bias);
        float p[4], q[4], g[4];
        load4<T>(pos, i, valid, vec, p);
        load4<T>(neg, i, valid, vec, q);
        load4<float>(grad, i, valid, vec, g);
#pragma unroll
        for (int k = 0; k < 4; k++) {
            p[k] = orn_inject_backward<N>(g[k], round_to_half(p[k]), b);
            q[k] = orn_inject_backward<N>(-g[k], round_to_half(q[k]), b);
        }
        store4(gp, i, valid, vec, p);
        store4(gn, i, valid, vec, q);
    }
};

template <typename T, int N> struct SingleFwd {
    const T *in; __half *out; const float *bias, *stdc; uint64_t seed, offset;
    __device__ __forceinline__ void apply(long long grp, long long i, int valid, bool vec) const
    {
        const Coef6 b = load_coef(bias), sd = load_coef(stdc);
        float s[4], z[4];
        load4<T>(in, i, valid, vec, s);
        normal4(seed, offset, (uint64_t)grp, 0u, z);
#pragma unroll
        for (int k = 0; k < 4; k++) s[k] = inject(orn_forward<N>(round_to_half(s[k])), z[k], b, sd);
        store4h(out, i, valid, vec, s);
    }
};

template <typename T, int N> struct SingleBwd {
    const float *grad; const T *in; float *gin; const float *bias;
    __device__ __forceinline__ void apply(long long, long long i, int valid, bool vec) const
    {
        const Coef6 b = load_coef(bias);
        float s[4], g[4];
        load4<T>(in, i, valid, vec, s);
        load4<float>(grad, i, valid, vec, g);
#pragma unroll
        for (int k = 0; k < 4; k++) g[k] = orn_inject_backward<N>(g[k], round_to_half(s[k]), b);
        store4(gin, i, valid, vec, g);
    }
};

template <typename OP> int run(const OP &op, long long n_elem, bool vec_ok, cudaStream_t st)
{
    if (n_elem == 0) return REXSC_OK;
    const long long n_groups = (n_elem + 3) >> 2;
    long long blocks = (n_groups + kPwThreads - 1) / kPwThreads;
    const long long cap = 148LL * 8 * 4; // a few waves of 8 resident CTAs per SM; grid-stride covers the rest
    if (blocks > cap) blocks = cap;
    pw_kernel<OP><<<(unsigned)blocks, kPwThreads, 0, st>>>(op, n_elem, vec_ok ? 1 : 0);
    REXSC_LAUNCH_CHECK("pw_kernel");
    return REXSC_OK;
}

inline bool aligned(const void *p, size_t a) { return (reinterpret_cast<uintptr_t>(p) % a) == 0; }
template <typename T> inline bool in_aligned(const void *p) { return aligned(p, V4<T>::kAlign); }

// dispatch over (dtype, n)
#define REXSC_PW_DISPATCH(DT, N, ...)                                                        \
    switch (DT) {                                                                             \
    case REXSC_F32: { using T = float; REXSC_PW_N(N, __VA_ARGS__) } break;                            \
    case REXSC_F16: { using T = __half; REXSC_PW_N(N, __VA_ARGS__) } break;                           \
    case REXSC_BF16: { using T = __nv_bfloat16; REXSC_PW_N(N, __VA_ARGS__) } break;                   \
    default: return REXSC_E_BAD_ARG;                                                          \
    }
#define REXSC_PW_N(N, ...)                                                                   \
    switch (N) {                                                                              \
    case 1: { constexpr int NN = 1; __VA_ARGS__ } break;                                             \
    case 2: { constexpr int NN = 2; __VA_ARGS__ } break;                                             \
    case 3: { constexpr int NN = 3; __VA_ARGS__ } break;                                             \
    case 4: { constexpr int NN = 4; __VA_ARGS__ } break;                                             \
    default: return REXSC_E_UNSUPPORTED;                                                      \
    }

} // namespace

} // namespace rexsc

using namespace rexsc;

extern "C" int rexsc_orn_fwd(const void *d_in, int32_t in_dtype, float *d_out, int64_t n_elem, int32_t or_n,
                             void *stream)
{
    if (n_elem < 0 || (n_elem > 0 && (!d_in || !d_out))) return REXSC_E_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    REXSC_PW_DISPATCH(in_dtype, or_n, {
        OrnFwd<T, NN> op{(const T *)d_in, d_out};
        return run(op, n_elem, in_aligned<T>(d_in) && aligned(d_out, 16), st);
    })
    return REXSC_E_BAD_ARG;
}

extern "C" int rexsc_orn_bwd(const float *d_grad_out, const void *d_in, int32_t in_dtype, float *d_grad_in,
                             int64_t n_elem, int32_t or_n, void *stream)
{
    if (n_elem < 0 || (n_elem > 0 && (!d_in || !d_grad_out || !d_grad_in))) return REXSC_E_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    REXSC_PW_DISPATCH(in_dtype, or_n, {
        OrnBwd<T, NN> op{d_grad_out, (const T *)d_in, d_grad_in};
        return run(op, n_elem, in_aligned<T>(d_in) && aligned(d_grad_out, 16) && aligned(d_grad_in, 16), st);
    })
    return REXSC_E_BAD_ARG;
}

extern "C" int rexsc_orn_bias_std_both_fwd(const void *d_pos, const void *d_neg, int32_t in_dtype,
                                           const float *d_bias_coef, const float *d_std_coef, float *d_out,
                                           int64_t n_elem, int32_t or_n, uint64_t seed, uint64_t offset, void *stream)
{
    if (n_elem < 0 || !d_bias_coef || !d_std_coef || (n_elem > 0 && (!d_pos || !d_neg || !d_out)))
        return REXSC_E_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    REXSC_PW_DISPATCH(in_dtype, or_n, {
        BothFwd<T, NN> op{(const T *)d_pos, (const T *)d_neg, d_out, d_bias_coef, d_std_coef, seed, offset};
        return run(op, n_elem, in_aligned<T>(d_pos) && in_aligned<T>(d_neg) && aligned(d_out, 16), st);
    })
    return REXSC_E_BAD_ARG;
}

extern "C" int rexsc_orn_bias_std_both_bwd(const float *d_grad_out, const void *d_pos, const void *d_neg,
                                           int32_t in_dtype, const float *d_bias_coef, float *d_grad_pos,
                                           float *d_grad_neg, int64_t n_elem, int32_t or_n, void *stream)
{
    if (n_elem < 0 || !d_bias_coef || (n_elem > 0 && (!d_pos || !d_neg || !d_grad_out || !d_grad_pos || !d_grad_neg)))
        return REXSC_E_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    REXSC_PW_DISPATCH(in_dtype, or_n, {
        BothBwd<T, NN> op{d_grad_out, (const T *)d_pos, (const T *)d_neg, d_grad_pos, d_grad_neg, d_bias_coef};
        return run(op, n_elem,
                   in_aligned<T>(d_pos) && in_aligned<T>(d_neg) && aligned(d_grad_out, 16) &&
                       aligned(d_grad_pos, 16) && aligned(d_grad_neg, 16),
                   st);
    })
    return REXSC_E_BAD_ARG;
}

extern "C" int rexsc_orn_bias_std_fwd(const void *d_in, int32_t in_dtype, const float *d_bias_coef,
                                      const float *d_std_coef, void *d_out_f16, int64_t n_elem, int32_t or_n,
                                      uint64_t seed, uint64_t offset, void *stream)
{
    if (n_elem < 0 || !d_bias_coef || !d_std_coef || (n_elem > 0 && (!d_in || !d_out_f16))) return REXSC_E_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    REXSC_PW_DISPATCH(in_dtype, or_n, {
        SingleFwd<T, NN> op{(const T *)d_in, (__half *)d_out_f16, d_bias_coef, d_std_coef, seed, offset};
        return run(op, n_elem, in_aligned<T>(d_in) && aligned(d_out_f16, 8), st);
    })
    return REXSC_E_BAD_ARG;
}

extern "C" int rexsc_orn_bias_std_bwd(const float *d_grad_out, const void *d_in, int32_t in_dtype,
                                      const float *d_bias_coef, float *d_grad_in, int64_t n_elem, int32_t or_n,
                                      void *stream)
{
    if (n_elem < 0 || !d_bias_coef || (n_elem > 0 && (!d_in || !d_grad_out || !d_grad_in))) return REXSC_E_BAD_ARG;
    cudaStream_t st = (cudaStream_t)stream;
    REXSC_PW_DISPATCH(in_dtype, or_n, {
        SingleBwd<T, NN> op{d_grad_out, (const T *)d_in, d_grad_in, d_bias_coef};
        return run(op, n_elem, in_aligned<T>(d_in) && aligned(d_grad_out, 16) && aligned(d_grad_in, 16), st);
    })
    return REXSC_E_BAD_ARG;
}
