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

// ---- packed fp32 pairs (Blackwell fma/mul/add.f32x2: two IEEE fp32 lanes per instruction) --------------------------
// Each lane rounds exactly like the scalar instruction, so a chain evaluated on pairs gives the same bits as the
// scalar functions above; it takes half the issue slots, which is what bounds the fused injection kernel.
typedef unsigned long long u64;
__device__ __forceinline__ u64 pk(float lo, float hi)
{
    u64 r;
    asm("mov.b64 %0, {%1, %2};" : "=l"(r) : "f"(lo), "f"(hi));
    return r;
}
__device__ __forceinline__ u64 pk1(float v) { return pk(v, v); }
__device__ __forceinline__ void upk(u64 v, float &lo, float &hi)
{
    asm("mov.b64 {%0, %1}, %2;" : "=f"(lo), "=f"(hi) : "l"(v));
}
__device__ __forceinline__ u64 fma2(u64 a, u64 b, u64 c)
{
    u64 d;
    asm("fma.rn.f32x2 %0, %1, %2, %3;" : "=l"(d) : "l"(a), "l"(b), "l"(c));
    return d;
}
__device__ __forceinline__ u64 mul2(u64 a, u64 b)
{
    u64 d;
    asm("mul.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ u64 add2(u64 a, u64 b)
{
    u64 d;
    asm("add.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ u64 sub2(u64 a, u64 b)
{
    u64 d;
    asm("sub.rn.f32x2 %0, %1, %2;" : "=l"(d) : "l"(a), "l"(b));
    return d;
}
__device__ __forceinline__ float sqrt_approx(float v)
{
    float r;
    asm("sqrt.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ float ex2_approx(float v)
{
    float r;
    asm("ex2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ float lg2_approx(float v)
{
    float r;
    asm("lg2.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ float sin_approx(float v)
{
    float r;
    asm("sin.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}
__device__ __forceinline__ float cos_approx(float v)
{
    float r;
    asm("cos.approx.ftz.f32 %0, %1;" : "=f"(r) : "f"(v));
    return r;
}

struct Coef6x2 { u64 c[6]; };  // every coefficient duplicated into both lanes
__device__ __forceinline__ Coef6x2 load_coef2(const float *p)
{
    Coef6x2 r;
#pragma unroll
    for (int i = 0; i < 6; i++) r.c[i] = pk1(__ldg(p + i));
    return r;
}

// orn_forward<N> on a pair.  fmaf(-a, e, x) is evaluated as fmaf(a, -e, x): the same product, the same rounding.
// e = 2^(s * -log2 e) through the hardware ex2 with denormals flushed.  __expf() differs from that only where its
// argument or result is denormal (|s| < 1e-38 or s > 87.3); there e contributes less than half an ulp of n to
// x = n - e * (...), so the forward value has the same bits either way (checked against the reference's kernels).
template <int N> __device__ __forceinline__ u64 orn_forward2(u64 s)
{
    float t0, t1;
    upk(mul2(s, pk1(-1.4426950408889634f)), t0, t1);
    const float e0 = ex2_approx(t0), e1 = ex2_approx(t1);
    if (N == 1) return pk(1.f - e0, 1.f - e1);
    const u64 ne = pk(-e0, -e1);
    u64 x = fma2(pk1((float)N), ne, pk1((float)N));
    if (N == 2) return fma2(s, ne, x);
    const u64 s2 = mul2(s, s);
    if (N == 3) {
        x = fma2(mul2(pk1(2.f), s), ne, x);
        return fma2(mul2(pk1(0.5f), s2), ne, x);
    }
    x = fma2(mul2(pk1(3.f), s), ne, x);
    const u64 s3 = mul2(s2, s);
    x = fma2(s2, ne, x);
    return fma2(mul2(pk1(1.f / 6.f), s3), ne, x);
}

// Mean x + B(x) and noise scale S(x) on a pair, both polynomials by Horner's rule.  Used only when noise is drawn:
// the result then agrees with the reference in distribution, not bit for bit, so the cheaper evaluation order is free.
__device__ __forceinline__ void inject_terms2_horner(u64 x, const Coef6x2 &b, const Coef6x2 &sd, u64 &mean, u64 &scale)
{
    u64 xb = fma2(b.c[5], x, b.c[4]);
    u64 xs = fma2(sd.c[5], x, sd.c[4]);
#pragma unroll
    for (int i = 3; i >= 0; i--) {
        xb = fma2(xb, x, b.c[i]);
        xs = fma2(xs, x, sd.c[i]);
    }
    mean = add2(x, xb);
    scale = xs;
}
// x + B(x) on a pair in the reference's operation order (powers, then fmaf chain): the bits of the scalar inject_terms
__device__ __forceinline__ u64 inject_mean2(u64 x, const Coef6x2 &b)
{
    const u64 x2 = mul2(x, x);
    u64 xb = fma2(b.c[1], x, b.c[0]);
    const u64 x3 = mul2(x2, x);
    xb = fma2(b.c[2], x2, xb);
    const u64 x4 = mul2(x3, x);
    xb = fma2(b.c[3], x3, xb);
    const u64 x5 = mul2(x4, x);
    xb = fma2(b.c[4], x4, xb);
    xb = fma2(b.c[5], x5, xb);
    return add2(x, xb);
}

// Philox4x32-10 with the ten round keys precomputed on the host (they depend on the seed only) and the two 32x32->64
// products written as such: two wide multiplies and two three-input XORs per round.
struct PhiloxKeys { uint32_t kx[10], ky[10]; };
__device__ __forceinline__ uint4 philox4x32_10_keyed(uint4 ctr, const PhiloxKeys &k)
{
#pragma unroll
    for (int r = 0; r < 10; r++) {
        const u64 p0 = (u64)0xD2511F53u * ctr.x;
        const u64 p1 = (u64)0xCD9E8D57u * ctr.z;
        ctr = make_uint4((uint32_t)(p1 >> 32) ^ ctr.y ^ k.kx[r], (uint32_t)p1, (uint32_t)(p0 >> 32) ^ ctr.w ^ k.ky[r],
                         (uint32_t)p0);
    }
    return ctr;
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

// ---- fused calibration + injection forward: eight elements per thread per iteration ------------------------------
template <typename T> struct V8;
template <> struct V8<float> {
    static __device__ __forceinline__ void load(const float *p, long long i, u64 (&v)[4])
    {
        const float4 a = __ldcs(reinterpret_cast<const float4 *>(p + i));
        const float4 b = __ldcs(reinterpret_cast<const float4 *>(p + i + 4));
        v[0] = pk(a.x, a.y); v[1] = pk(a.z, a.w); v[2] = pk(b.x, b.y); v[3] = pk(b.z, b.w);
    }
};
template <> struct V8<__half> {
    static __device__ __forceinline__ void load(const __half *p, long long i, u64 (&v)[4])
    {
        const uint4 t = __ldcs(reinterpret_cast<const uint4 *>(p + i));
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int k = 0; k < 4; k++) {
            const float2 f = __half22float2(*reinterpret_cast<const __half2 *>(&w[k]));
            v[k] = pk(f.x, f.y);
        }
    }
};
template <> struct V8<__nv_bfloat16> {
    static __device__ __forceinline__ void load(const __nv_bfloat16 *p, long long i, u64 (&v)[4])
    {
        const uint4 t = __ldcs(reinterpret_cast<const uint4 *>(p + i));
        const uint32_t w[4] = {t.x, t.y, t.z, t.w};
#pragma unroll
        for (int k = 0; k < 4; k++) v[k] = pk(__uint_as_float(w[k] << 16), __uint_as_float(w[k] & 0xffff0000u));
    }
};

// Octets [0, n_oct) go through the packed path (128-bit loads, coefficients in registers, noise skipped when every std
// coefficient is zero); the elements behind them (and everything when the pointers are not 16-byte aligned) take the
// 4-element path of BothFwd::apply.
//
// Noise of the packed path: one Philox4x32-10 block per octet (counter = octet index, stream tag 1; the 4-element path
// uses tag 0, so the two never share a counter).  Each 32-bit word feeds one Box-Muller pair: its low half is the
// radius uniform, its high half the angle, 16 bits each -- radii up to 4.8 sigma on a 65536-step grid, which the
// mean / variance / kurtosis checks cannot tell from 32-bit uniforms and which halves the generator's cost.  The
// pair's two normals go to two adjacent elements.  The reference draws S(xp)*e1 - S(xn)*e2 with two normals per
// element; the difference of two independent Gaussians is one Gaussian of variance S(xp)^2 + S(xn)^2, so one draw
// per element gives the same output distribution: noise = sqrt((S(xp)^2 + S(xn)^2) * (-2 ln u)) * {sin, cos}(angle).
template <typename T, int N, bool NOISY>
__device__ __forceinline__ void both_fwd_octets(const BothFwd<T, N> &op, long long n_oct, const PhiloxKeys &keys)
{
    const Coef6x2 b = load_coef2(op.bias);
    Coef6x2 sd;
    if (NOISY) sd = load_coef2(op.stdc);
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x; o < n_oct; o += stride) {
        const long long i = o << 3;
        u64 p[4], q[4];
        V8<T>::load(op.pos, i, p);
        V8<T>::load(op.neg, i, q);
        uint32_t w[4];
        if (NOISY) {
            const uint4 r = philox4x32_10_keyed(
                make_uint4((uint32_t)o, (uint32_t)(o >> 32), (uint32_t)op.offset, ((uint32_t)(op.offset >> 32) << 1) | 1u),
                keys);
            w[0] = r.x; w[1] = r.y; w[2] = r.z; w[3] = r.w;
        }
        float r8[8];
#pragma unroll
        for (int k = 0; k < 4; k++) {
            u64 res;
            if (NOISY) {
                u64 mp, sp, mn, sn;
                inject_terms2_horner(orn_forward2<N>(p[k]), b, sd, mp, sp);
                inject_terms2_horner(orn_forward2<N>(q[k]), b, sd, mn, sn);
                // 16-bit fields dropped into the mantissa of a float in [1, 2): no integer-to-float conversion
                const float fu = __uint_as_float(0x3f800000u | ((w[k] << 7) & 0x007fff80u));
                const float fa = __uint_as_float(0x3f800000u | ((w[k] >> 9) & 0x007fff80u));
                const float u = fu - (1.0f - 7.62939453125e-06f);                       // (j + 0.5) / 65536 in (0, 1)
                const float ang = fmaf(fa, 6.2831853071795865f, -9.42477796f + 4.79e-05f); // (-pi, pi)
                const float rr = -1.3862943611198906f * lg2_approx(u);                  // -2 ln u
                float v0, v1;
                upk(mul2(fma2(sp, sp, mul2(sn, sn)), pk1(rr)), v0, v1);
                res = fma2(pk(sqrt_approx(v0), sqrt_approx(v1)), pk(sin_approx(ang), cos_approx(ang)), sub2(mp, mn));
            } else {
                res = sub2(inject_mean2(orn_forward2<N>(p[k]), b), inject_mean2(orn_forward2<N>(q[k]), b));
            }
            upk(res, r8[2 * k], r8[2 * k + 1]);
        }
        __stcs(reinterpret_cast<float4 *>(op.out + i), make_float4(r8[0], r8[1], r8[2], r8[3]));
        __stcs(reinterpret_cast<float4 *>(op.out + i + 4), make_float4(r8[4], r8[5], r8[6], r8[7]));
    }
}

// The exact path (every std coefficient zero) as a function of its own: it needs more registers than the noisy loop
// (the reference's evaluation order keeps five powers alive), and out of line its spills stay out of that loop.
template <typename T, int N>
__device__ __noinline__ void both_fwd_quiet(const BothFwd<T, N> &op, long long n_oct, const PhiloxKeys &keys)
{
    both_fwd_octets<T, N, false>(op, n_oct, keys);
}

// The kernel is bound by instruction issue, not by HBM (about 45 instructions per element with noise); what it needs
// is many resident warps to cover the XU latencies, hence small CTAs and a tight register budget.
template <typename T> struct BothFwdCfg { static constexpr int kThreads = 128, kMinBlocks = sizeof(T) == 2 ? 12 : 8; };

template <typename T, int N>
__global__ void __launch_bounds__(BothFwdCfg<T>::kThreads, BothFwdCfg<T>::kMinBlocks)
both_fwd_kernel(BothFwd<T, N> op, long long n_oct, const __grid_constant__ PhiloxKeys keys)
{
    bool noisy = false;
#pragma unroll
    for (int k = 0; k < 6; k++) noisy |= (__ldg(op.stdc + k) != 0.f);
    if (!noisy) {
        both_fwd_quiet<T, N>(op, n_oct, keys);
        return;
    }
    both_fwd_octets<T, N, true>(op, n_oct, keys);
}

// Groups [first, n_groups) of four elements through BothFwd::apply with scalar accesses: the up to seven elements
// behind the last octet, or the whole tensor when a pointer is not 16-byte aligned.
template <typename T, int N>
__global__ void __launch_bounds__(kPwThreads) both_fwd_tail_kernel(BothFwd<T, N> op, long long first, long long n_groups,
                                                                   long long n_elem)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long g = first + (long long)blockIdx.x * blockDim.x + threadIdx.x; g < n_groups; g += stride) {
        const long long i = g << 2;
        const int valid = (int)(n_elem - i < 4 ? n_elem - i : 4);
        op.apply(g, i, valid, false);
    }
}

template <typename T, int N> int run_both_fwd(const BothFwd<T, N> &op, long long n_elem, bool vec_ok, cudaStream_t st)
{
    if (n_elem == 0) return REXSC_OK;
    constexpr int kThreads = BothFwdCfg<T>::kThreads;
    const long long n_oct = vec_ok ? (n_elem >> 3) : 0;
    if (n_oct > 0) {
        long long blocks = (n_oct + kThreads - 1) / kThreads;
        const long long cap = 148LL * BothFwdCfg<T>::kMinBlocks * 8;  // eight waves of resident CTAs; the loop covers the rest
        if (blocks > cap) blocks = cap;
        PhiloxKeys keys;
        uint32_t kx = (uint32_t)op.seed, ky = (uint32_t)(op.seed >> 32);
        for (int r = 0; r < 10; r++) {
            keys.kx[r] = kx;
            keys.ky[r] = ky;
            kx += 0x9E3779B9u;
            ky += 0xBB67AE85u;
        }
        both_fwd_kernel<T, N><<<(unsigned)blocks, kThreads, 0, st>>>(op, n_oct, keys);
        REXSC_LAUNCH_CHECK("both_fwd_kernel");
    }
    const long long first = n_oct << 1, n_groups = (n_elem + 3) >> 2;
    if (first < n_groups) {
        long long blocks = (n_groups - first + kPwThreads - 1) / kPwThreads;
        if (blocks > 148LL * 32) blocks = 148LL * 32;
        both_fwd_tail_kernel<T, N><<<(unsigned)blocks, kPwThreads, 0, st>>>(op, first, n_groups, n_elem);
        REXSC_LAUNCH_CHECK("both_fwd_tail_kernel");
    }
    return REXSC_OK;
}

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

// ---- OR-n activation forward, eight elements per thread on packed pairs ---------------------------------------------
// Same values as OrnFwd::apply (orn_forward2 keeps the scalar chain's bits); fewer instructions per element, which is
// what bounds this kernel at 6 bytes per element (fp16 in, fp32 out).
template <typename T, int N>
__global__ void __launch_bounds__(256) orn_fwd_octets_kernel(const T *__restrict__ in, float *__restrict__ out, long long n_oct)
{
    const long long stride = (long long)gridDim.x * blockDim.x;
    for (long long o = (long long)blockIdx.x * blockDim.x + threadIdx.x; o < n_oct; o += stride) {
        const long long i = o << 3;
        u64 p[4];
        V8<T>::load(in, i, p);
        float r[8];
#pragma unroll
        for (int k = 0; k < 4; k++) upk(orn_forward2<N>(p[k]), r[2 * k], r[2 * k + 1]);
        __stcs(reinterpret_cast<float4 *>(out + i), make_float4(r[0], r[1], r[2], r[3]));
        __stcs(reinterpret_cast<float4 *>(out + i + 4), make_float4(r[4], r[5], r[6], r[7]));
    }
}

template <typename T, int N> int run_orn_fwd(const T *in, float *out, long long n_elem, bool vec16, cudaStream_t st)
{
    if (n_elem == 0) return REXSC_OK;
    const long long n_oct = vec16 ? (n_elem >> 3) : 0;
    if (n_oct > 0) {
        long long blocks = (n_oct + 255) / 256;
        if (blocks > 148LL * 8 * 4) blocks = 148LL * 8 * 4;
        orn_fwd_octets_kernel<T, N><<<(unsigned)blocks, 256, 0, st>>>(in, out, n_oct);
        REXSC_LAUNCH_CHECK("orn_fwd_octets_kernel");
    }
    const long long done = n_oct << 3;
    if (done < n_elem) { // the up to seven elements behind the last octet, or everything when a pointer is misaligned
        OrnFwd<T, N> op{in + done, out + done};
        const bool vec = (reinterpret_cast<uintptr_t>(in + done) % V4<T>::kAlign) == 0 &&
                         (reinterpret_cast<uintptr_t>(out + done) % 16) == 0;
        return run(op, n_elem - done, vec, st);
    }
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
        return run_orn_fwd<T, NN>((const T *)d_in, d_out, n_elem, aligned(d_in, 16) && aligned(d_out, 16), st);
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
        return run_both_fwd(op, n_elem, aligned(d_pos, 16) && aligned(d_neg, 16) && aligned(d_out, 16), st);
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
