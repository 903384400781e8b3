// FXP saturating conv, closed form, on the 5th-generation tensor cores (tcgen05, int8 -> int32 in TMEM).
//
// Valid exactly where fxp_conv.cu's closed form is (plain add, no shift, operands <= 127): per sign the
// reference's sequential saturating adder equals  min( sum a*w + sum (a&1)(w&1), 2^pmax ), every addend is
// non-negative, so splitting K into MMA steps cannot change where the sum saturates -- the cap is applied once to
// the finished int32 accumulator (the host checks that K*127*127 + K cannot overflow it).
//
// Implicit GEMM:  D[m][n'] = sum_k' A[m][k'] * B[n'][k'],  k' runs over the products twice (values, then parity
// bits), n' over the output channels of the CTA's chunk twice (positive weights, then negative weights).  CTA = 128
// output pixels (TMEM lanes) x up to 256 columns.  The products are ordered (tap, channel) with the channels padded
// to a multiple of 16 -- the order does not matter to the closed form -- and the int8 activations are kept pixel-major
// (NHWC, same channel padding), so 16 consecutive k' of an output pixel are 16 consecutive bytes in memory.
//   * producers (all 128 threads): fetch the int8 activation slab (128 rows x 128 bytes of k') as eight 16-byte
//     loads per row through a chunk -> tensor-offset table, and copy the prepacked weight slab, both written to
//     shared memory in the 128-byte swizzled K-major layout the MMA's shared-memory descriptors name;
//   * one thread issues tcgen05.mma.kind::i8 (M=128, N=N', K=32) four times per slab and commits to an mbarrier;
//   * epilogue: tcgen05.ld 32 lanes x 32 columns per warp, min(., cap), pos - neg, coalesced NCHW int32 stores.
// Every mbarrier wait is bounded; on a time-out the CTA records it, frees its TMEM and returns.
#include "common.cuh"

namespace rexsc {

namespace {

constexpr int kUmmaM = 128;          // output pixels per CTA = TMEM lanes
constexpr int kSlabBytes = 128;      // k' bytes per pipeline step (one 128-byte swizzle row)
constexpr int kUmmaK = 32;           // int8 elements per MMA instruction
constexpr uint32_t kUmmaWaitLimit = 1u << 22;

struct UmmaArgs {
    int N, C, Hp, Wp, Co, OH, OW, sh, sw;
    int H, W, ph, pw; // unpadded activation and the op's zero padding (operand preparation)
    float scale;      // 2^precision_in
    int Cp;          // channels padded to 16 (pixel pitch of the int8 activations, channel pitch of k')
    int Kp;          // k' extent padded to kSlabBytes (values + parity)
    int CB, CBp;     // output channels per CTA chunk, padded to 8
    int CBq;         // first MMA column of the negative-weight block (CBp rounded up to 32: aligned TMEM reads)
    int NP;          // MMA N: positive block [0, CBp), negative block [CBq, CBq + CBp), padded to 16
    int tmem_cols;   // power of two >= NP, >= 32
    int cap;
    long long M;
};

__device__ __forceinline__ uint32_t smem_addr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// shared-memory matrix descriptor: K-major, 128-byte swizzle, 8-row groups 1024 bytes apart
__device__ __forceinline__ uint64_t umma_desc_k_sw128(uint32_t saddr)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3fff);       // start address, 16-byte units
    d |= (uint64_t)1 << 16;                       // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024 >> 4) << 32;             // stride byte offset between 8-row groups
    d |= (uint64_t)1 << 46;                       // descriptor version (Blackwell)
    d |= (uint64_t)2 << 61;                       // layout type: 128-byte swizzle
    return d;
}

// byte offset of 16-byte chunk `c` (0..7) of row `r` inside a [rows][128 B] tile with 128-byte swizzle
__device__ __forceinline__ uint32_t sw128_offset(int r, int c) { return (uint32_t)(r * 128 + ((c ^ (r & 7)) << 4)); }

// Unswizzled ("interleaved") K-major alternative: the tile is stored as 16-byte K-columns, [chunk][row][16 B], so
// every row of a K-column sits 16 bytes after the previous one (8-row core matrices back to back, stride byte
// offset 128) and the next K-column starts `rows * 16` bytes later (leading byte offset).
__device__ __forceinline__ uint64_t umma_desc_k_interleaved(uint32_t saddr, uint32_t rows)
{
    uint64_t d = 0;
    d |= (uint64_t)((saddr >> 4) & 0x3fff);
    d |= (uint64_t)(((rows * 16) >> 4) & 0x3fff) << 16; // leading byte offset: next 16-byte K-column
    d |= (uint64_t)(128 >> 4) << 32;                    // stride byte offset: next 8-row core matrix
    d |= (uint64_t)1 << 46;
    return d;                                           // layout type 0: no swizzle
}
__device__ __forceinline__ uint32_t interleaved_offset(int r, int c, int rows) { return (uint32_t)((c * rows + r) * 16); }

__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity)
{
    for (uint32_t i = 0; i < kUmmaWaitLimit; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    return false;
}

// PREFETCH_B: also fetch the weight slab one step ahead (64 more registers: two CTAs per SM instead of four) -- pays
// on grids of at most a wave or two of CTAs, whose time is one CTA's chain of slabs
template <bool SWIZZLED, bool PREFETCH_B>
__global__ void __launch_bounds__(128, PREFETCH_B ? 2 : 6)
fxp_conv_umma_kernel(UmmaArgs a, const int8_t *__restrict__ act, const int8_t *__restrict__ wpk,
                     const int32_t *__restrict__ koff, int32_t *__restrict__ out, int *__restrict__ status)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // the swizzled operand tiles must start on a 1024-byte boundary of the shared window
    uint8_t *smem = smem_raw + ((1024u - (smem_addr(smem_raw) & 1023u)) & 1023u);
    uint8_t *a_s = smem;                                   // 128 rows x 128 B
    uint8_t *b_s = smem + kUmmaM * kSlabBytes;             // NP rows x 128 B (1024-byte aligned: 16 KB offset)
    uint64_t *bar = reinterpret_cast<uint64_t *>(b_s + a.NP * kSlabBytes);        // (the launch sizes the tile by NP)
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);

    const int tid = threadIdx.x, warp = tid >> 5;
    const long long m = (long long)blockIdx.x * kUmmaM + tid;
    const int chunk = blockIdx.y;
    const bool row_live = m < a.M;
    long long abase = 0;
    int ow = 0, oh = 0, n = 0;
    if (row_live) {
        ow = (int)(m % a.OW);
        long long t = m / a.OW;
        oh = (int)(t % a.OH);
        n = (int)(t / a.OH);
        abase = (((long long)n * a.Hp + (long long)oh * a.sh) * a.Wp + (long long)ow * a.sw) * a.Cp;
    }

    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(smem_addr(bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_addr(tmem_slot)),
                     "r"((uint32_t)a.tmem_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // instruction descriptor: int32 accumulate, signed int8 A and B, both K-major, N = NP, M = 128
    const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(a.NP >> 3) << 17) | ((uint32_t)(kUmmaM >> 4) << 24);
    const int8_t *wchunk = wpk + (size_t)chunk * a.NP * a.Kp;
    const int n_slabs = a.Kp / kSlabBytes;
    bool failed = false;

    // The activation words of a slab are fetched into registers one slab ahead: the loads of slab s + 1 are in flight
    // while the tensor core works through slab s (the shared-memory tiles are single: they are rewritten once those
    // MMAs are done).  Row = this thread's output pixel, 8 chunks of 16 k' each = 16 channels of one tap.  Weight
    // slab: NP rows x 8 chunks of the prepacked weights, chunk i * 128 + tid for i < 16 (NP <= 256).
    uint4 av[8], bv[PREFETCH_B ? 16 : 1];
    auto load_slab = [&](int slab) {
#pragma unroll
        for (int c = 0; c < 8; c++) {
            av[c] = make_uint4(0u, 0u, 0u, 0u);
            const int off = __ldg(koff + slab * 8 + c);         // < 0: padding; bit 30 set: parity operand
            if (row_live && off >= 0) {
                av[c] = __ldg(reinterpret_cast<const uint4 *>(act + abase + (off & 0x3fffffff)));
                if (off & 0x40000000) {
                    av[c].x &= 0x01010101u; av[c].y &= 0x01010101u; av[c].z &= 0x01010101u; av[c].w &= 0x01010101u;
                }
            }
        }
        if (PREFETCH_B) {
#pragma unroll
            for (int i = 0; i < (PREFETCH_B ? 16 : 1); i++) {
                const int e = i * 128 + tid, r = e >> 3, c = e & 7;
                if (e < a.NP * 8)
                    bv[i] = __ldg(reinterpret_cast<const uint4 *>(wchunk + (size_t)r * a.Kp + slab * kSlabBytes) + c);
            }
        }
    };
    load_slab(0);
    for (int slab = 0; slab < n_slabs; slab++) {
#pragma unroll
        for (int c = 0; c < 8; c++)
            *reinterpret_cast<uint4 *>(a_s + (SWIZZLED ? sw128_offset(tid, c) : interleaved_offset(tid, c, kUmmaM))) = av[c];
        if (PREFETCH_B) {
#pragma unroll
            for (int i = 0; i < (PREFETCH_B ? 16 : 1); i++) {
                const int e = i * 128 + tid, r = e >> 3, c = e & 7;
                if (e < a.NP * 8)
                    *reinterpret_cast<uint4 *>(b_s + (SWIZZLED ? sw128_offset(r, c) : interleaved_offset(r, c, a.NP))) = bv[i];
            }
        }
        // B slab without prefetch: NP rows x 8 chunks, straight copy of the prepacked weights (L2-resident)
        for (int i = tid; !PREFETCH_B && i < a.NP * 8; i += blockDim.x) {
            const int r = i >> 3, c = i & 7;
            const uint4 v = __ldg(reinterpret_cast<const uint4 *>(wchunk + (size_t)r * a.Kp + slab * kSlabBytes) + c);
            *reinterpret_cast<uint4 *>(b_s + (SWIZZLED ? sw128_offset(r, c) : interleaved_offset(r, c, a.NP))) = v;
        }
        // generic-proxy writes must be visible to the tensor core's async-proxy reads
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            const uint64_t da = SWIZZLED ? umma_desc_k_sw128(smem_addr(a_s)) : umma_desc_k_interleaved(smem_addr(a_s), kUmmaM);
            const uint64_t db = SWIZZLED ? umma_desc_k_sw128(smem_addr(b_s)) : umma_desc_k_interleaved(smem_addr(b_s), a.NP);
#pragma unroll
            for (int kk = 0; kk < kSlabBytes / kUmmaK; kk++) {
                const uint32_t accumulate = (slab > 0 || kk > 0) ? 1u : 0u;
                // advancing K by 32 bytes: +2 address units (16 B) inside a swizzle row, or two K-columns further
                // in the interleaved layout
                const uint64_t dak = da + (uint64_t)(SWIZZLED ? kk * (kUmmaK >> 4) : kk * 2 * (kUmmaM * 16 >> 4));
                const uint64_t dbk = db + (uint64_t)(SWIZZLED ? kk * (kUmmaK >> 4) : kk * 2 * (a.NP * 16 >> 4));
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "setp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                    ::"r"(tmem_base), "l"(dak), "l"(dbk), "r"(idesc), "r"(accumulate), "r"(0u)
                    : "memory");
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(
                             smem_addr(bar))
                         : "memory");
        }
        if (slab + 1 < n_slabs) load_slab(slab + 1);
        // the slab buffers are reused next step: wait until the MMAs that read them have completed
        if (!mbar_wait(smem_addr(bar), (uint32_t)(slab & 1))) failed = true;
        failed = __syncthreads_or(failed ? 1 : 0) != 0;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (failed) break;
    }

    if (!failed) {
        // ---- epilogue: this warp reads its 32 TMEM lanes, 32 columns at a time ---------------------------------
        const uint32_t lane_base = (uint32_t)(warp * 32) << 16;
        const size_t ohw = (size_t)a.OH * a.OW;
        for (int c0 = 0; c0 < a.CBp; c0 += 32) {
            uint32_t vp[32], vn[32];
            const uint32_t tp = tmem_base + lane_base + (uint32_t)c0;
            const uint32_t tn = tmem_base + lane_base + (uint32_t)(a.CBq + c0);
            // both reads start on a multiple of 32 columns and stay inside the allocation (tmem_cols >= 2 * CBq);
            // columns at or past CB carry zero weights and are masked below
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(vp[0]), "=r"(vp[1]), "=r"(vp[2]), "=r"(vp[3]), "=r"(vp[4]), "=r"(vp[5]), "=r"(vp[6]), "=r"(vp[7]),
                  "=r"(vp[8]), "=r"(vp[9]), "=r"(vp[10]), "=r"(vp[11]), "=r"(vp[12]), "=r"(vp[13]), "=r"(vp[14]),
                  "=r"(vp[15]), "=r"(vp[16]), "=r"(vp[17]), "=r"(vp[18]), "=r"(vp[19]), "=r"(vp[20]), "=r"(vp[21]),
                  "=r"(vp[22]), "=r"(vp[23]), "=r"(vp[24]), "=r"(vp[25]), "=r"(vp[26]), "=r"(vp[27]), "=r"(vp[28]),
                  "=r"(vp[29]), "=r"(vp[30]), "=r"(vp[31])
                : "r"(tp) : "memory");
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(vn[0]), "=r"(vn[1]), "=r"(vn[2]), "=r"(vn[3]), "=r"(vn[4]), "=r"(vn[5]), "=r"(vn[6]), "=r"(vn[7]),
                  "=r"(vn[8]), "=r"(vn[9]), "=r"(vn[10]), "=r"(vn[11]), "=r"(vn[12]), "=r"(vn[13]), "=r"(vn[14]),
                  "=r"(vn[15]), "=r"(vn[16]), "=r"(vn[17]), "=r"(vn[18]), "=r"(vn[19]), "=r"(vn[20]), "=r"(vn[21]),
                  "=r"(vn[22]), "=r"(vn[23]), "=r"(vn[24]), "=r"(vn[25]), "=r"(vn[26]), "=r"(vn[27]), "=r"(vn[28]),
                  "=r"(vn[29]), "=r"(vn[30]), "=r"(vn[31])
                : "r"(tn) : "memory");
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
            if (row_live) {
#pragma unroll
                for (int j = 0; j < 32; j++) {
                    const int cl = c0 + j;
                    const int co = chunk * a.CB + cl;
                    if (cl < a.CB && co < a.Co) {
                        const int p = min((int)vp[j], a.cap), q = min((int)vn[j], a.cap);
                        out[((size_t)n * a.Co + co) * ohw + (size_t)oh * a.OW + ow] = p - q;
                    }
                }
            }
        }
    } else if (tid == 0) {
        atomicExch(status, 3);
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)a.tmem_cols)
                     : "memory");
    }
}

// ---- operand preparation ------------------------------------------------------------------------------------
// Both kernels quantise on the fly (round-half-even of value * 2^p, fixed_cuda.cpp:28-30: activations clamped to
// [0, 2^p - 1], weights split into a positive and a negative magnitude), so the tensor-core path needs two launches
// before the conv kernel instead of four.
// k' = tap * Cp + c for the values, K2 + tap * Cp + c for the parity bits (K2 = KH * KW * Cp); weights are [co][c][tap]
template <typename T>
__global__ void fxp_umma_pack_kernel(UmmaArgs a, int KH, int KW, int n_chunks, const T *__restrict__ w,
                                     int8_t *__restrict__ wpk, int32_t *__restrict__ koff)
{
    const int KHW = KH * KW, K2 = KHW * a.Cp;
    // weights: wpk[chunk][row n' in 0..NP)[k' in 0..Kp), row = sign * CBq + local channel
    const long long total = (long long)n_chunks * a.NP * a.Kp;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        const int kp = (int)(i % a.Kp);
        const long long r = i / a.Kp;
        const int row = (int)(r % a.NP);
        const int chunk = (int)(r / a.NP);
        const int sign = row >= a.CBq ? 1 : 0, cl = row - sign * a.CBq;
        const int co = chunk * a.CB + cl;
        int v = 0;
        if (cl < a.CB && co < a.Co && kp < 2 * K2) {
            const int k = kp < K2 ? kp : kp - K2;
            const int tap = k / a.Cp, c = k - tap * a.Cp;
            if (c < a.C) {
                const float x = load_as_float<T>(w, ((long long)co * a.C + c) * KHW + tap) * a.scale;
                v = sign ? (int)rintf(-fminf(fmaxf(x, 1.f - a.scale), 0.f)) : (int)rintf(fminf(fmaxf(x, 0.f), a.scale - 1.f));
                if (kp >= K2) v &= 1;
            }
        }
        wpk[i] = (int8_t)v;
    }
    // 16-byte chunk of k' -> byte offset of its 16 channels inside the int8 activations, relative to tap (0,0) of the
    // output pixel
    for (int j = blockIdx.x * blockDim.x + threadIdx.x; j < a.Kp / 16; j += gridDim.x * blockDim.x) {
        const int kp = j * 16;
        int off = -1;
        if (kp < 2 * K2) {
            const int k = kp < K2 ? kp : kp - K2;
            const int tap = k / a.Cp, cg = k - tap * a.Cp, kh = tap / KW, kw = tap - kh * KW;
            off = (kh * a.Wp + kw) * a.Cp + cg;
            if (kp >= K2) off |= 0x40000000;
        }
        koff[j] = off;
    }
}

// dense NCHW activations -> zero-padded int8 NHWC with the channels padded to Cp; one thread per padded pixel and 16
// channels
template <typename T>
__global__ void fxp_umma_act_kernel(UmmaArgs a, const T *__restrict__ x, int8_t *__restrict__ q8)
{
    const int groups = a.Cp / 16;
    const long long plane = (long long)a.Hp * a.Wp, total = (long long)a.N * plane * groups;
    for (long long i = (long long)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (long long)gridDim.x * blockDim.x) {
        // consecutive threads take consecutive pixels of one channel group: the strided reads coalesce
        const long long pix = i % plane;
        const long long t = i / plane;
        const int g = (int)(t % groups), n = (int)(t / groups);
        const int h = (int)(pix / a.Wp), wq = (int)(pix - (long long)h * a.Wp);
        const int hi = h - a.ph, wi = wq - a.pw;
        uint32_t w[4] = {0u, 0u, 0u, 0u};
        if (hi >= 0 && hi < a.H && wi >= 0 && wi < a.W) {
#pragma unroll
            for (int b = 0; b < 16; b++) {
                const int c = g * 16 + b;
                if (c < a.C) {
                    const float v = load_as_float<T>(x, (((long long)n * a.C + c) * a.H + hi) * a.W + wi) * a.scale;
                    const int q = (int)rintf(fminf(fmaxf(v, 0.f), a.scale - 1.f));
                    w[b >> 2] |= (uint32_t)(q & 0xff) << (8 * (b & 3));
                }
            }
        }
        *reinterpret_cast<uint4 *>(q8 + ((long long)n * plane + pix) * a.Cp + g * 16) = make_uint4(w[0], w[1], w[2], w[3]);
    }
}

} // namespace

static long long umma_k2(int C, long long K) // padded product count per operand kind: taps x padded channels
{
    const long long khw = C > 0 ? K / C : 0;
    return khw * ((C + 15) / 16 * 16);
}

size_t fxp_umma_workspace_bytes(int N, int C, int Hp, int Wp, int Co, long long K)
{
    const int CB = Co < 128 ? Co : 128;
    const int n_chunks = (Co + CB - 1) / CB;
    const int Cp = (C + 15) / 16 * 16;
    const long long Kp = (2 * umma_k2(C, K) + kSlabBytes - 1) / kSlabBytes * kSlabBytes;
    return align_up((size_t)N * Hp * Wp * Cp, 256) + align_up((size_t)n_chunks * 256 * Kp, 256) +
           align_up((size_t)Kp * 4, 256);
}

bool fxp_umma_supported(int C, int Hp, int Wp, long long K)
{
    // the offset table keeps an in-image byte offset in 30 bits
    return (long long)((C + 15) / 16 * 16) * Hp * Wp < (1LL << 30) && 2 * umma_k2(C, K) <= (1 << 20);
}

int launch_fxp_conv_umma(int N, int C, int H, int W, int ph, int pw, int Co, int KH, int KW, int OH, int OW, int sh,
                         int sw, int cap, float scale, const void *d_act, int act_dtype, const void *d_w, int w_dtype,
                         void *ws, int32_t *out, int *status, bool swizzled, cudaStream_t st)
{
    UmmaArgs a;
    const int Hp = H + 2 * ph, Wp = W + 2 * pw;
    const long long K = (long long)C * KH * KW;
    a.N = N; a.C = C; a.Hp = Hp; a.Wp = Wp; a.Co = Co; a.OH = OH; a.OW = OW; a.sh = sh; a.sw = sw;
    a.H = H; a.W = W; a.ph = ph; a.pw = pw; a.scale = scale;
    a.Cp = (C + 15) / 16 * 16;
    a.Kp = (int)((2 * umma_k2(C, K) + kSlabBytes - 1) / kSlabBytes * kSlabBytes);
    a.CB = Co < 128 ? Co : 128;
    a.CBp = (a.CB + 7) / 8 * 8;
    a.CBq = (a.CBp + 31) / 32 * 32;
    a.NP = (a.CBq + a.CBp + 15) / 16 * 16;
    a.tmem_cols = 32;
    while (a.tmem_cols < 2 * a.CBq) a.tmem_cols *= 2; // the epilogue reads whole 32-column groups of both blocks
    if (a.tmem_cols > 512 || a.NP > 256) return REXSC_E_UNSUPPORTED;
    a.cap = cap;
    a.M = (long long)N * OH * OW;
    const int n_chunks = (Co + a.CB - 1) / a.CB;
    uint8_t *w8 = static_cast<uint8_t *>(ws);
    int8_t *q8 = reinterpret_cast<int8_t *>(w8);
    int8_t *wpk = reinterpret_cast<int8_t *>(w8 + align_up((size_t)N * Hp * Wp * a.Cp, 256));
    int32_t *koff = reinterpret_cast<int32_t *>(reinterpret_cast<uint8_t *>(wpk) +
                                                align_up((size_t)n_chunks * a.NP * a.Kp, 256));
    const long long n_act = (long long)N * Hp * Wp * (a.Cp / 16); // one thread per pixel and 16 channels
    const unsigned ab = (unsigned)((n_act + 255) / 256 < 148 * 16 ? (n_act + 255) / 256 : 148 * 16);
    switch (act_dtype) {
    case REXSC_F32: fxp_umma_act_kernel<float><<<ab, 256, 0, st>>>(a, (const float *)d_act, q8); break;
    case REXSC_F16: fxp_umma_act_kernel<__half><<<ab, 256, 0, st>>>(a, (const __half *)d_act, q8); break;
    default: fxp_umma_act_kernel<__nv_bfloat16><<<ab, 256, 0, st>>>(a, (const __nv_bfloat16 *)d_act, q8); break;
    }
    REXSC_LAUNCH_CHECK("fxp_umma_act_kernel");
    switch (w_dtype) {
    case REXSC_F32: fxp_umma_pack_kernel<float><<<148 * 4, 256, 0, st>>>(a, KH, KW, n_chunks, (const float *)d_w, wpk, koff); break;
    case REXSC_F16: fxp_umma_pack_kernel<__half><<<148 * 4, 256, 0, st>>>(a, KH, KW, n_chunks, (const __half *)d_w, wpk, koff); break;
    default:
        fxp_umma_pack_kernel<__nv_bfloat16><<<148 * 4, 256, 0, st>>>(a, KH, KW, n_chunks, (const __nv_bfloat16 *)d_w, wpk, koff);
        break;
    }
    REXSC_LAUNCH_CHECK("fxp_umma_pack_kernel");
    // operand tiles sized by the layer: narrow layers fit more CTAs per SM, which is what hides their load latency
    const size_t smem = (size_t)kUmmaM * kSlabBytes + (size_t)a.NP * kSlabBytes + 64 + 1024;
    dim3 grid((unsigned)((a.M + kUmmaM - 1) / kUmmaM), (unsigned)n_chunks);
    const bool few_ctas = (long long)grid.x * grid.y <= 2 * 148;
    auto kernel = swizzled ? (few_ctas ? fxp_conv_umma_kernel<true, true> : fxp_conv_umma_kernel<true, false>)
                           : (few_ctas ? fxp_conv_umma_kernel<false, true> : fxp_conv_umma_kernel<false, false>);
    REXSC_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    kernel<<<grid, 128, smem, st>>>(a, q8, wpk, koff, out, status);
    REXSC_LAUNCH_CHECK("fxp_conv_umma_kernel");
    return REXSC_OK;
}

} // namespace rexsc
