// SC conv forward on the 5th-generation tensor cores (tcgen05, int8 operands, int32 accumulators in TMEM).
//
// Per time slot t the count that OR-n saturates is a plain contraction of 0/1 values,
//     count_t[pixel][sign, co] = sum_{tap, c} a_t[pixel + tap][c] * w_t[sign, co][tap, c],
// and only min(count_t, n) is non-linear -- it is applied to the finished accumulator of every slot:
//     out[pixel][sign, co] = sum_t min(count_t, n)            (sc_device.cu:127-151 of the reference).
// So every slot is one int8 GEMM, M = 128 stored-grid positions (TMEM lanes), N = 128 (64 output channels x
// {positive, negative} weight stream), K = taps x channels, issued as tcgen05.mma.kind::i8 M128 N128 K32.
//
// Operands are generated in shared memory from bit planes (one bit per element and slot, 32 channels per word):
//   A_t  the slot's activation bits of the tile's patch, expanded to bytes as 16-byte K-columns
//        [16-channel column][patch row][16 B] (unswizzled K-major).  Rows sit 16 bytes apart, so the operand of
//        filter tap (kh, kw) is the SAME buffer with its start address moved by tap_offset rows: no im2col.
//   B_t  the slot's weight bits, [tap][16-channel column][128 rows][16 B].
// The M dimension runs over consecutive positions of the stored (padded) pixel grid; positions that are not the
// origin of an output pixel produce rows that are computed and dropped.
//
// One CTA = 256 threads: everybody expands operands, one thread issues the MMAs and commits to an mbarrier, then
// the eight warps read TMEM (warp w: lanes 32*(w%4).., columns 64*(w/4)..), clamp to n and add into 16-bit packed
// running sums.  Two CTAs share an SM, so one CTA's expansion / epilogue overlaps the other's MMAs.
// Every wait is bounded; on a time-out the CTA reports through the status word, frees its TMEM and returns.
#include "common.cuh"

namespace rexsc {

namespace {

constexpr int kTcThreads = 256;
constexpr int kTcM = 256;          // stored-grid positions per CTA: two MMA row blocks that share one weight operand
constexpr int kTcSub = 128;        // rows of one MMA (TMEM lanes)
constexpr int kTcCout = 64;        // output channels per CTA
constexpr int kTcN = 2 * kTcCout;  // MMA N: positive block [0,64), negative block [64,128)
constexpr int kTcMaxTaps = 9;      // filter taps whose weight operand is staged at once
constexpr uint32_t kTcWaitLimit = 1u << 22;

struct TcArgs {
    int OH, OW, sh, sw, KH, KW, KHW, Co, CW, CK;
    int nrh, Wq, Hrows, Wrow, max_tap;
    int rows_a;      // patch rows staged per slot: kTcM + max_tap, rounded up to 8
    int slots, n_or;
    long long NHW, NHWp;
    int out_nhwc;
};

__device__ __forceinline__ uint32_t saddr(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// unswizzled K-major descriptor: rows 16 B apart (8-row core matrices back to back), K-columns `lbo_bytes` apart
__device__ __forceinline__ uint64_t desc_interleaved(uint32_t addr, uint32_t lbo_bytes)
{
    uint64_t d = 0;
    d |= (uint64_t)((addr >> 4) & 0x3fff);
    d |= (uint64_t)((lbo_bytes >> 4) & 0x3fff) << 16;
    d |= (uint64_t)(128 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    return d;
}

__device__ __forceinline__ bool tc_wait(uint32_t bar, uint32_t parity)
{
    for (uint32_t i = 0; i < kTcWaitLimit; i++) {
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

// 16 bits -> 16 bytes of 0/1 (bit i -> byte i)
__device__ __forceinline__ uint4 spread16(uint32_t h)
{
    uint4 r;
    r.x = ((h & 0xfu) * 0x00204081u) & 0x01010101u;
    r.y = (((h >> 4) & 0xfu) * 0x00204081u) & 0x01010101u;
    r.z = (((h >> 8) & 0xfu) * 0x00204081u) & 0x01010101u;
    r.w = (((h >> 12) & 0xfu) * 0x00204081u) & 0x01010101u;
    return r;
}

#define REXSC_TMEM_LD32(arr, taddr)                                                                                   \
    asm volatile(                                                                                                     \
        "tcgen05.ld.sync.aligned.32x32b.x32.b32 "                                                                     \
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "                                     \
        "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"                     \
        : "=r"(arr[0]), "=r"(arr[1]), "=r"(arr[2]), "=r"(arr[3]), "=r"(arr[4]), "=r"(arr[5]), "=r"(arr[6]),           \
          "=r"(arr[7]), "=r"(arr[8]), "=r"(arr[9]), "=r"(arr[10]), "=r"(arr[11]), "=r"(arr[12]), "=r"(arr[13]),       \
          "=r"(arr[14]), "=r"(arr[15]), "=r"(arr[16]), "=r"(arr[17]), "=r"(arr[18]), "=r"(arr[19]), "=r"(arr[20]),    \
          "=r"(arr[21]), "=r"(arr[22]), "=r"(arr[23]), "=r"(arr[24]), "=r"(arr[25]), "=r"(arr[26]), "=r"(arr[27]),    \
          "=r"(arr[28]), "=r"(arr[29]), "=r"(arr[30]), "=r"(arr[31])                                                  \
        : "r"(taddr)                                                                                                  \
        : "memory")

// 32 TMEM columns as 16 registers: the low 16 bits of two adjacent columns per register
#define REXSC_TMEM_LD16_PACKED(arr, taddr)                                                                            \
    asm volatile(                                                                                                     \
        "tcgen05.ld.sync.aligned.32x32b.x16.pack::16b.b32 "                                                           \
        "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15}, [%16];"                              \
        : "=r"(arr[0]), "=r"(arr[1]), "=r"(arr[2]), "=r"(arr[3]), "=r"(arr[4]), "=r"(arr[5]), "=r"(arr[6]),           \
          "=r"(arr[7]), "=r"(arr[8]), "=r"(arr[9]), "=r"(arr[10]), "=r"(arr[11]), "=r"(arr[12]), "=r"(arr[13]),       \
          "=r"(arr[14]), "=r"(arr[15])                                                                                \
        : "r"(taddr)                                                                                                  \
        : "memory")

__global__ void __launch_bounds__(kTcThreads, 2)
sc_conv_tc_kernel(TcArgs a, const uint32_t *__restrict__ Ab, const uint32_t *__restrict__ Wb,
                  int16_t *__restrict__ out_pos, int16_t *__restrict__ out_neg, int *__restrict__ status)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((128u - (saddr(smem_raw) & 127u)) & 127u);
    uint8_t *a_s = smem;                                            // [4][rows_a][16]
    uint8_t *b_s = a_s + 4 * a.rows_a * 16;                         // [KHW][4][128][16]
    uint64_t *bar = reinterpret_cast<uint64_t *>(b_s + a.KHW * 4 * kTcN * 16);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bar + 1);
    int *tap_s = reinterpret_cast<int *>(tmem_slot + 1);

    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const long long q0 = (long long)blockIdx.x * kTcM; // first stored-grid position of the tile
    const int nc = blockIdx.y;                         // 64-channel output chunk

    if (tid < a.KHW) {
        const int kh = tid / a.KW, kw = tid - kh * a.KW;
        tap_s[tid] = tap_offset(kh, kw, a.sh, a.sw, a.nrh, a.Wrow, a.Wq);
    }
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(saddr(bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(tmem_slot)),
                     "r"((uint32_t)(2 * kTcN)) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // instruction descriptor: int32 accumulators, signed int8 operands, both K-major, N = 128, M = 128
    const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTcN >> 3) << 17) | ((uint32_t)(kTcSub >> 4) << 24);
    const uint32_t a_lbo = (uint32_t)a.rows_a * 16, b_lbo = kTcN * 16;
    const int wrow_words = a.KHW * a.CW;               // words per weight row and slot
    const uint32_t *Wchunk = Wb + (size_t)nc * a.slots * kTcN * wrow_words;

    // running sums: this thread owns row block warp/4, TMEM lane 32*(warp%4)+lane and all 128 columns of that block,
    // two 16-bit sums per register (column pairs as the packed TMEM load delivers them)
    uint32_t acc[64];
#pragma unroll
    for (int j = 0; j < 64; j++) acc[j] = 0u;
    const uint32_t my_taddr = tmem_base + ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)((warp >> 2) * kTcN);
    const uint32_t n2 = (uint32_t)a.n_or | ((uint32_t)a.n_or << 16);

    // Bit words of one pipeline step (slot, 64-channel chunk) are fetched into registers one step ahead, so
    // that their L2 latency hides behind the previous step's MMAs.
    //   weights: thread -> (row = tid & 127, word half = tid >> 7), one word per filter tap
    //   patch:   thread -> rows tid and tid + 256, both words of the chunk
    const int w_row = tid & (kTcN - 1), w_half = tid >> 7;
    uint32_t wbits[kTcMaxTaps], abits[4];
    auto load_bits = [&](int step) {
        const int s = step / a.CK, ck = step - s * a.CK;
        const int cw = 2 * ck + w_half;
        const uint32_t *src = Wchunk + ((size_t)s * kTcN + w_row) * wrow_words + cw;
#pragma unroll
        for (int tap = 0; tap < kTcMaxTaps; tap++)
            wbits[tap] = (tap < a.KHW && cw < a.CW) ? __ldg(src + tap * a.CW) : 0u;
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int r = tid + kTcThreads * j;
            const long long P = q0 + r;
#pragma unroll
            for (int h = 0; h < 2; h++) {
                const int cwa = 2 * ck + h;
                abits[2 * j + h] = (r < a.rows_a && P < a.NHW && cwa < a.CW)
                                       ? __ldg(Ab + ((size_t)s * a.CW + cwa) * a.NHWp + P) : 0u;
            }
        }
    };
    auto expand_bits = [&]() {
#pragma unroll
        for (int tap = 0; tap < kTcMaxTaps; tap++) {
            if (tap < a.KHW) {
                uint8_t *dst = b_s + ((size_t)(tap * 4 + 2 * w_half) * kTcN + w_row) * 16;
                *reinterpret_cast<uint4 *>(dst) = spread16(wbits[tap]);
                *reinterpret_cast<uint4 *>(dst + kTcN * 16) = spread16(wbits[tap] >> 16);
            }
        }
#pragma unroll
        for (int j = 0; j < 2; j++) {
            const int r = tid + kTcThreads * j;
            if (r < a.rows_a) {
#pragma unroll
                for (int h = 0; h < 2; h++) {
                    *reinterpret_cast<uint4 *>(a_s + ((size_t)(2 * h) * a.rows_a + r) * 16) = spread16(abits[2 * j + h]);
                    *reinterpret_cast<uint4 *>(a_s + ((size_t)(2 * h + 1) * a.rows_a + r) * 16) = spread16(abits[2 * j + h] >> 16);
                }
            }
        }
    };
    // count -> min(count, n) -> running sums for the slot whose accumulators are complete in TMEM
    auto slot_epilogue = [&]() {
#pragma unroll
        for (int g = 0; g < 4; g++) {
            uint32_t v[16];
            REXSC_TMEM_LD16_PACKED(v, my_taddr + (uint32_t)(g * 32));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int j = 0; j < 16; j++) acc[g * 16 + j] += __vminu2(v[j], n2);
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };

    bool failed = false;
    const int n_steps = a.slots * a.CK;
    const uint64_t da0 = desc_interleaved(saddr(a_s), a_lbo), db0 = desc_interleaved(saddr(b_s), b_lbo);
    load_bits(0);
    for (int step = 0; step < n_steps; step++) {
        const int s = step / a.CK, ck = step - s * a.CK;
        expand_bits(); // the operand buffers are free: the previous step's MMAs were waited for
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
        __syncthreads();
        if (tid == 0) {
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            // the start-address field counts 16-byte units from bit 0, i.e. operand rows: moving an operand by
            // rows / K-columns is an integer add on the descriptor
#pragma unroll
            for (int sub = 0; sub < kTcM / kTcSub; sub++) {
                const uint32_t d_addr = tmem_base + (uint32_t)(sub * kTcN);
                for (int tap = 0; tap < a.KHW; tap++) {
#pragma unroll
                    for (int kk = 0; kk < 2; kk++) {
                        if (2 * ck + kk >= a.CW) break; // no channels in this half of the chunk
                        const uint64_t da = da0 + (uint64_t)(uint32_t)(sub * kTcSub + tap_s[tap] + 2 * kk * a.rows_a);
                        const uint64_t db = db0 + (uint64_t)(uint32_t)((tap * 4 + 2 * kk) * kTcN);
                        const uint32_t accumulate = (ck > 0 || tap > 0 || kk > 0) ? 1u : 0u;
                        asm volatile(
                            "{\n\t.reg .pred p;\n\t"
                            "setp.ne.b32 p, %4, 0;\n\t"
                            "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                            ::"r"(d_addr), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
                            : "memory");
                    }
                }
            }
            asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(saddr(bar))
                         : "memory");
        }
        // while the tensor core works: fetch the next step's bits
        if (step + 1 < n_steps) load_bits(step + 1);
        if (!tc_wait(saddr(bar), (uint32_t)(step & 1))) failed = true;
        failed = __syncthreads_or(failed ? 1 : 0) != 0;
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (failed) break;
        if (ck == a.CK - 1) slot_epilogue(); // the next slot's first MMA comes after the next barrier
    }

    if (!failed) {
        // ---- store: row = one stored-grid position; it is an output pixel iff it is the tap-(0,0) origin of one ----
        const long long q = q0 + (warp >> 2) * kTcSub + (warp & 3) * 32 + lane;
        if (q < a.NHW) {
            const int colp = (int)(q % a.Wrow);
            const long long t = q / a.Wrow;
            const int rowp = (int)(t % a.Hrows);
            const long long n = t / a.Hrows;
            const int oh = rowp / a.nrh;
            if (colp < a.OW && rowp % a.nrh == 0 && oh < a.OH) {
                const int co0 = nc * kTcCout;
                const size_t ohw = (size_t)a.OH * a.OW;
                const size_t m = ((size_t)n * a.OH + oh) * a.OW + colp;
                // acc[0..31] = positive block (columns 0..63), acc[32..63] = negative block
#pragma unroll
                for (int sign = 0; sign < 2; sign++) {
                    int16_t *dst = sign ? out_neg : out_pos;
                    const uint32_t *av = acc + sign * 32;
                    if (a.out_nhwc) {
                        int16_t *row = dst + m * a.Co + co0;
                        if ((a.Co & 7) == 0 && co0 + kTcCout <= a.Co) {
#pragma unroll
                            for (int j = 0; j < 32; j += 4)
                                *reinterpret_cast<uint4 *>(row + 2 * j) = make_uint4(av[j], av[j + 1], av[j + 2], av[j + 3]);
                        } else {
#pragma unroll
                            for (int j = 0; j < 64; j++)
                                if (co0 + j < a.Co) row[j] = (int16_t)((av[j >> 1] >> (16 * (j & 1))) & 0xffffu);
                        }
                    } else {
#pragma unroll
                        for (int j = 0; j < 64; j++)
                            if (co0 + j < a.Co)
                                dst[((size_t)n * a.Co + co0 + j) * ohw + (size_t)oh * a.OW + colp] =
                                    (int16_t)((av[j >> 1] >> (16 * (j & 1))) & 0xffffu);
                    }
                }
            }
        }
    } else if (tid == 0) {
        atomicExch(status, 4);
    }

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)(2 * kTcN))
                     : "memory");
}

// ---- bit planes --------------------------------------------------------------------------------------------
// activation words A[wd][c][P] (bit t = slot 32*wd + t)  ->  Ab[slot][cw][P] (bit b = channel 32*cw + b)
__global__ void __launch_bounds__(256) bitplane_act_kernel(const uint32_t *__restrict__ A, uint32_t *__restrict__ Ab,
                                                           int Cpad, int CW, long long NHWp, long long a_plane_words)
{
    __shared__ uint32_t tile[32][33]; // [channel][pixel]
    __shared__ uint32_t outp[32][33]; // [slot][pixel]
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const long long P0 = (long long)blockIdx.x * 32;
    const int cw = blockIdx.y, wd = blockIdx.z;
    const uint32_t *Aw = A + (size_t)wd * a_plane_words;
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int cl = warp + 8 * i, c = cw * 32 + cl;
        uint32_t v = 0;
        if (c < Cpad && P0 + lane < NHWp) v = Aw[(size_t)c * NHWp + P0 + lane];
        tile[cl][lane] = v;
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int p = warp + 8 * i;
        const uint32_t v = tile[lane][p]; // lane = channel
        uint32_t mine = 0;
#pragma unroll
        for (int t = 0; t < 32; t++) {
            const uint32_t b = __ballot_sync(0xffffffffu, (v >> t) & 1u);
            if (lane == t) mine = b;
        }
        outp[lane][p] = mine; // lane = slot
    }
    __syncthreads();
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const int t = warp + 8 * i;
        if (P0 + lane < NHWp) Ab[((size_t)(wd * 32 + t) * CW + cw) * NHWp + P0 + lane] = outp[t][lane];
    }
}

// weight words + signs (layout of the ALU kernels)  ->  Wb[nchunk][slot][row][tap*CW + cw],
// row = sign*64 + local output channel, bit b = channel 32*cw + b
__global__ void __launch_bounds__(256) bitplane_weight_kernel(const uint32_t *__restrict__ Wt, const uint32_t *__restrict__ S,
                                                              uint32_t *__restrict__ Wb, int Co, int C, int KHW, int CCH,
                                                              int CW, int words, int NC, long long w_plane_words)
{
    // one warp per (nchunk, wd, row, tap, cw); lane = channel
    const long long gw = ((long long)blockIdx.x * blockDim.x + threadIdx.x) >> 5;
    const int lane = threadIdx.x & 31;
    const long long total = (long long)NC * words * kTcN * KHW * CW;
    if (gw >= total) return;
    long long t = gw;
    const int cw = (int)(t % CW); t /= CW;
    const int tap = (int)(t % KHW); t /= KHW;
    const int row = (int)(t % kTcN); t /= kTcN;
    const int wd = (int)(t % words);
    const int nchunk = (int)(t / words);
    const int sign = row >> 6, col = row & 63;
    const int co = nchunk * kTcCout + col;
    const int c = cw * 32 + lane;
    uint32_t v = 0;
    if (co < Co && c < C) {
        const int nt = co / kTileN, nl = co % kTileN, cch = c / kChunkC, cc = c % kChunkC;
        const size_t blk = ((size_t)nt * CCH + cch) * KHW + tap;
        const uint32_t sg = S[blk * (kTileN / kWarpN) + nl / kWarpN];
        const int neg = (sg >> (cc * kWarpN + nl % kWarpN)) & 1u;
        if (neg == sign) v = Wt[(size_t)wd * w_plane_words + (blk * kChunkC + cc) * kTileN + nl];
    }
    uint32_t mine = 0;
#pragma unroll
    for (int tt = 0; tt < 32; tt++) {
        const uint32_t b = __ballot_sync(0xffffffffu, (v >> tt) & 1u);
        if (lane == tt) mine = b;
    }
    const int slots = words * 32;
    Wb[(((size_t)nchunk * slots + wd * 32 + lane) * kTcN + row) * ((size_t)KHW * CW) + tap * CW + cw] = mine;
}

// Tensor-pipe issue-rate probe: back-to-back int8 MMAs (M128 x N x K32) on fixed shared-memory operands.
__global__ void __launch_bounds__(128, 2) mma_probe_kernel(int iters, int n_cols, uint32_t *sink)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    uint8_t *smem = smem_raw + ((128u - (saddr(smem_raw) & 127u)) & 127u);
    uint8_t *a_s = smem;                 // [2][128][16]
    uint8_t *b_s = smem + 2 * 128 * 16;  // [2][n_cols][16]
    __shared__ uint64_t bar;
    __shared__ uint32_t tmem_slot;
    const int tid = threadIdx.x, warp = tid >> 5;
    for (int i = tid; i < (2 * 128 * 16 + 2 * n_cols * 16) / 16; i += blockDim.x)
        reinterpret_cast<uint4 *>(smem)[i] = make_uint4(0x01010101u, 0x01010101u, 0x01010101u, 0x01010101u);
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], 1;" ::"r"(saddr(&bar)) : "memory");
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(&tmem_slot)),
                     "r"((uint32_t)n_cols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = tmem_slot;
    const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(n_cols >> 3) << 17) | ((uint32_t)(128 >> 4) << 24);
    bool ok = true;
    if (tid == 0) {
        const uint64_t da = desc_interleaved(saddr(a_s), 128 * 16), db = desc_interleaved(saddr(b_s), (uint32_t)n_cols * 16);
        uint32_t phase = 0;
        for (int it = 0; it < iters && ok; it++) {
#pragma unroll
            for (int j = 0; j < 16; j++) {
                const uint32_t accumulate = (it > 0 || j > 0) ? 1u : 0u;
                asm volatile(
                    "{\n\t.reg .pred p;\n\t"
                    "setp.ne.b32 p, %4, 0;\n\t"
                    "tcgen05.mma.cta_group::1.kind::i8 [%0], %1, %2, %3, {%5, %5, %5, %5}, p;\n\t}"
                    ::"r"(tmem_base), "l"(da), "l"(db), "r"(idesc), "r"(accumulate), "r"(0u)
                    : "memory");
            }
            // commit and wait every 64 iterations so that the queue stays full but bounded
            if ((it & 63) == 63 || it == iters - 1) {
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(saddr(&bar))
                             : "memory");
                ok = tc_wait(saddr(&bar), phase & 1u);
                phase++;
            }
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t v[16];
    REXSC_TMEM_LD16_PACKED(v, tmem_base + ((uint32_t)(warp * 32) << 16));
    asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
    sink[blockIdx.x * blockDim.x + tid] = v[0] + (ok ? 0u : 0x80000000u);
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0)
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)n_cols) : "memory");
}

size_t tc_smem_bytes(const ConvPlan &p)
{
    const int rows_a = (kTcM + p.max_tap + 7) / 8 * 8;
    return (size_t)4 * rows_a * 16 + (size_t)p.KHW * 4 * kTcN * 16 + 8 + 8 + kTcMaxTaps * 4 + 128;
}

} // namespace

int launch_mma_probe(int blocks, int iters, int n_cols, uint32_t *d_sink, cudaStream_t st)
{
    if (blocks < 1 || iters < 1 || (n_cols != 128 && n_cols != 256) || !d_sink) return REXSC_E_BAD_ARG;
    const size_t smem = 2 * 128 * 16 + 2 * (size_t)n_cols * 16 + 128;
    mma_probe_kernel<<<blocks, 128, smem, st>>>(iters, n_cols, d_sink);
    REXSC_LAUNCH_CHECK("mma_probe_kernel");
    return REXSC_OK;
}

bool conv_tc_supported(const ConvPlan &p)
{
    if (p.n_or < 1) return false;
    if (p.KHW > kTcMaxTaps) return false;
    if (tc_smem_bytes(p) > 112 * 1024) return false;                          // two CTAs per SM
    if (kTcM + p.max_tap > 2 * kTcThreads) return false;                      // patch rows: two per thread
    const long long cap = p.n_or < p.Kdot ? p.n_or : p.Kdot;                   // largest per-slot contribution
    if ((long long)p.words * 32 * cap > 65535) return false;                  // 16-bit running sums
    if (p.Kdot > (1 << 24)) return false;
    if ((p.NHW + kTcM - 1) / kTcM > 0x7fffffffLL) return false;
    return true;
}

size_t conv_tc_workspace_bytes(const ConvPlan &p)
{
    const int CW = (p.C + 31) / 32, NC = (p.Co + kTcCout - 1) / kTcCout;
    const size_t ab = (size_t)p.words * 32 * CW * p.NHWp * 4;
    const size_t wb = (size_t)NC * p.words * 32 * kTcN * p.KHW * CW * 4;
    return align_up(ab, 256) + align_up(wb, 256);
}

// stream words of the ALU layout -> bit planes (part of the expand stage when the tensor kernel is selected)
int launch_tc_bitplanes(const ConvPlan &p, const uint32_t *d_A, const uint32_t *d_Wt, const uint32_t *d_S,
                        void *d_tc_ws, cudaStream_t st)
{
    if (!conv_tc_supported(p)) return REXSC_E_UNSUPPORTED;
    const int CW = (p.C + 31) / 32, NC = (p.Co + kTcCout - 1) / kTcCout;
    const int slots = p.words * 32;
    uint32_t *Ab = static_cast<uint32_t *>(d_tc_ws);
    uint32_t *Wb = reinterpret_cast<uint32_t *>(static_cast<uint8_t *>(d_tc_ws) +
                                                align_up((size_t)slots * CW * p.NHWp * 4, 256));
    {
        dim3 grid((unsigned)((p.NHWp + 31) / 32), (unsigned)CW, (unsigned)p.words);
        bitplane_act_kernel<<<grid, 256, 0, st>>>(d_A, Ab, p.Cpad, CW, p.NHWp, p.a_plane_words);
        REXSC_LAUNCH_CHECK("bitplane_act_kernel");
    }
    {
        const long long warps = (long long)NC * p.words * kTcN * p.KHW * CW;
        bitplane_weight_kernel<<<(unsigned)((warps * 32 + 255) / 256), 256, 0, st>>>(d_Wt, d_S, Wb, p.Co, p.C, p.KHW, p.CCH, CW,
                                                                                     p.words, NC, p.w_plane_words);
        REXSC_LAUNCH_CHECK("bitplane_weight_kernel");
    }
    return REXSC_OK;
}

int launch_conv_tc(const ConvPlan &p, const rexsc_sc_conv_desc &d, void *d_tc_ws, int16_t *d_pos, int16_t *d_neg,
                   int *d_status, cudaStream_t st)
{
    if (!conv_tc_supported(p)) return REXSC_E_UNSUPPORTED;
    const int CW = (p.C + 31) / 32, NC = (p.Co + kTcCout - 1) / kTcCout;
    const int slots = p.words * 32;
    const uint32_t *Ab = static_cast<const uint32_t *>(d_tc_ws);
    const uint32_t *Wb = reinterpret_cast<const uint32_t *>(static_cast<const uint8_t *>(d_tc_ws) +
                                                            align_up((size_t)slots * CW * p.NHWp * 4, 256));
    TcArgs a;
    a.OH = p.OH; a.OW = p.OW; a.sh = p.sh; a.sw = p.sw; a.KH = p.KH; a.KW = p.KW; a.KHW = p.KHW; a.Co = p.Co;
    a.CW = CW; a.CK = (CW + 1) / 2;
    a.nrh = p.nrh; a.Wq = p.Wq; a.Hrows = p.Hrows; a.Wrow = p.Wrow; a.max_tap = p.max_tap;
    a.rows_a = (kTcM + p.max_tap + 7) / 8 * 8;
    a.slots = slots; a.n_or = p.n_or;
    a.NHW = p.NHW; a.NHWp = p.NHWp; a.out_nhwc = d.out_channels_last;
    const size_t smem = tc_smem_bytes(p);
    REXSC_CUDA_CHECK(cudaFuncSetAttribute(sc_conv_tc_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem));
    dim3 grid((unsigned)((p.NHW + kTcM - 1) / kTcM), (unsigned)NC);
    sc_conv_tc_kernel<<<grid, kTcThreads, smem, st>>>(a, Ab, Wb, d_pos, d_neg, d_status);
    REXSC_LAUNCH_CHECK("sc_conv_tc_kernel");
    return REXSC_OK;
}

} // namespace rexsc
