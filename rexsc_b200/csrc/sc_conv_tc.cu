// SC conv forward on the 5th-generation tensor cores (tcgen05, int8 operands, int32 accumulators in TMEM).
//
// Per time slot t the count that OR-n saturates is a plain contraction of 0/1 values,
//     count_t[pixel][sign, co] = sum_{tap, c} a_t[pixel + tap][c] * w_t[sign, co][tap, c],
// and only min(count_t, n) is non-linear -- it is applied to the finished accumulator of every slot:
//     out[pixel][sign, co] = sum_t min(count_t, n)            (sc_device.cu:127-151 of the reference).
// So every slot is one int8 GEMM, M = output-pixel candidates (TMEM lanes, 128 per MMA), N = 128 (64 output
// channels x {positive, negative} weight stream), K = taps x channels, issued as tcgen05.mma.kind::i8 M128 N128 K32.
//
// Rows.  The M dimension runs over the "origin grid": per image Ho x Wo candidates (i, j), candidate (i, j) being
// the padded-input pixel (i*stride_h, j*stride_w), i.e. the top-left tap of output pixel (i, j) when i < OH and
// j < OW (other rows are computed and dropped; they are the padding of the grid, a few percent).  A CTA owns 256
// consecutive candidates.
//
// Operands are generated in shared memory from bit planes (one bit per element and slot, 32 channels per word):
//   A_t  the slot's activation bits of the tile's patch as 16-byte K-columns [16-channel column][patch row][16 B]
//        (unswizzled K-major, rows 16 bytes apart).  The patch is kept as one plane per stride residue
//        (kh % stride_h, kw % stride_w); inside a plane, row r holds the pixel of that residue that belongs to
//        candidate o0 + r.  The operand of filter tap (kh, kw) is then the SAME buffer with its start address moved
//        to plane(kh % sh, kw % sw) + (kh / sh) * Wo + kw / sw rows: no im2col, for any stride.
//   B_t  the slot's weight bits, [tap][16-channel column][128 rows][16 B].
// Operand bytes are 0 or a power of two (see kTcMaskA), the accumulators hold 8 * count.
//
// One persistent CTA per SM walks its tiles as a single pipeline (a tile's first loads and its store overlap the
// neighbouring tiles' MMAs): 16 warps expand operands and fold counts, 2 warps issue MMAs (one per 128-row block; a single
// thread cannot keep the tensor core busy with 128-column MMAs).  A pipeline step is one slot x one chunk of 32 or
// 64 channels.  Operand buffers and accumulators are double-buffered and every dependence is an mbarrier phase:
// while the tensor core works through step i, the expanding warps write the operands of step i+1, fold the slot
// that finished, and already hold the bit words of step i+2 in registers.
// Every wait is bounded; on a time-out the CTA reports through the status word, frees its TMEM and returns.
#include "common.cuh"
#include <stdlib.h>
#include <type_traits>

namespace rexsc {

namespace {

constexpr int kTcWorkers = 512;             // threads that expand operands and fold counts
constexpr int kTcThreads = kTcWorkers + 64; // + two warps that only issue MMAs, one per 128-row block
constexpr int kTcM = 256;          // candidates per CTA: two MMA row blocks that share one weight operand
constexpr int kTcSub = 128;        // rows of one MMA (TMEM lanes)
constexpr int kTcCout = 64;        // output channels per CTA
constexpr int kTcN = 2 * kTcCout;  // MMA N: positive block [0,64), negative block [64,128)
constexpr int kTcMaxTaps = 9;      // filter taps whose weight operand is staged at once
constexpr int kTcMaxARows = 3;     // patch rows per expanding thread (all residue planes together)
constexpr int kTcMaxBWords = 5;    // weight words per expanding thread and step
constexpr int kTcPrefetch = 4;     // pipeline steps between the L2 prefetch of patch bits and their use
constexpr uint32_t kTcWaitLimit = 1u << 18; // try_wait attempts before a wait gives up (each may sleep kTcSuspendNs)
constexpr uint32_t kTcSuspendNs = 4000;    // a waiting warp sleeps in the barrier unit instead of spinning on issue slots

struct TcArgs {
    int OH, OW, KHW, Co, CW;
    int KWc;         // 32-channel words per pipeline step: 2, or 1 when shared memory is short
    int CK;          // pipeline steps per slot = ceil(CW / KWc)
    int nrh, nrw, Wq, Hrows, Wrow; // stored pixel grid (see tap_offset in common.cuh)
    int Ho, Wo;      // origin grid of one image
    int shift;       // candidates by which the patch starts BEFORE the tile's first candidate: 0, or Wo + 1 on the
                     // compact grid (ConvPlan::origin), whose candidates are the CENTRE taps of their output pixels
    int Mh;          // patch rows per residue plane: kTcM + largest in-plane tap shift, rounded up to 8
    int rows_a;      // patch rows of all planes
    int slots, n_or;
    long long total_o; // candidates = N * Ho * Wo
    int tiles_x;       // candidate tiles = ceil(total_o / kTcM)
    int total_tiles;   // tiles_x * (64-channel output chunks); tile index = chunk * tiles_x + x
    int out_vec;       // both output pointers are 16-byte aligned: rows may be stored as 128-bit vectors
    int balanced;      // 0: a CTA walks whole tiles blockIdx.x, + gridDim.x, ...
                       // 1: the (tile, time slot) pairs, in that order, are cut into gridDim.x equal runs, one per CTA.
                       //    A tile that two or more CTAs share is zeroed before the launch (zero_shared_tiles_kernel)
                       //    and every sharer adds its partial sums with packed 16-bit atomics; tiles that lie inside
                       //    one run are stored plainly.  No SM idles in a last, partly filled wave of tiles.
                       // 2: the same runs for outputs whose rows cannot take packed adds (NCHW, ragged or unaligned
                       //    channel runs): the host clears the whole outputs and every tile adds 16-bit values.
    long long NHWp;
    int out_nhwc;
    int descale_each; // 1: running sums would overflow 16 bits in accumulator units, so every slot is descaled
    int tap_off[kTcMaxTaps]; // patch-row offset of every tap (kernel parameters are warp-uniform by construction)
};

// the tiles and time slots of CTA b of G (TcArgs::balanced)
struct TileRun {
    int first_tile, tile_stride, tiles; // tile k of the CTA = first_tile + k * tile_stride
    int slot_first;                     // first time slot of its first tile
    int slot_last_end;                  // end (exclusive) of the time slots of its last tile
    int slots;                          // time slots of all its tiles together
};

__host__ __device__ __forceinline__ TileRun tile_run(int total_tiles, int slots, int balanced, int b, int G)
{
    TileRun r;
    if (!balanced) {
        r.first_tile = b; r.tile_stride = G;
        r.tiles = (total_tiles - b + G - 1) / G;
        r.slot_first = 0; r.slot_last_end = slots;
        r.slots = r.tiles * slots;
    } else {
        // run b = units [u0, u1) of the total_tiles * slots (tile, slot) pairs; G <= units, so no run is empty
        const long long units = (long long)total_tiles * slots;
        const long long u0 = units * b / G, u1 = units * (b + 1) / G;
        const long long last = (u1 - 1) / slots;
        r.first_tile = (int)(u0 / slots); r.tile_stride = 1;
        r.tiles = (int)(last - r.first_tile) + 1;
        r.slot_first = (int)(u0 - (long long)r.first_tile * slots);
        r.slot_last_end = (int)(u1 - 1 - last * slots) + 1;
        r.slots = (int)(u1 - u0);
    }
    return r;
}

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
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2, %3;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}"
            : "=r"(ok) : "r"(bar), "r"(parity), "r"(kTcSuspendNs) : "memory");
        if (ok) return true;
    }
    return false;
}

// Operand bytes are not 0/1.  Expanding bit i of a nibble to byte i costs one byte-replicate (PRMT) and one AND when
// the byte keeps its bit where it was: patch bytes are 0 or 2^i (mask 0x08040201).  The weight bit planes store each
// nibble bit-reversed and use mask 0x01020408, so their bytes are 0 or 2^(3-i); every coincidence contributes
// 2^i * 2^(3-i) = 8 and the accumulators hold 8 * count.
constexpr uint32_t kTcMaskA = 0x08040201u, kTcMaskW = 0x01020408u;
constexpr int kTcScaleLog2 = 3;
constexpr uint32_t kDescaleMask = (0xffffu >> kTcScaleLog2) * 0x00010001u; // after a packed 16-bit shift right

// 32 bits -> two groups of 16 operand bytes (bits 0..15 and 16..31; byte i <- bit i)
template <uint32_t MASK>
__device__ __forceinline__ void spread32(uint32_t h, uint4 &lo16, uint4 &hi16)
{
    const uint32_t g = h >> 4; // high nibbles moved into the low half of each byte
    lo16.x = __byte_perm(h, 0, 0x0000) & MASK;
    lo16.y = __byte_perm(g, 0, 0x0000) & MASK;
    lo16.z = __byte_perm(h, 0, 0x1111) & MASK;
    lo16.w = __byte_perm(g, 0, 0x1111) & MASK;
    hi16.x = __byte_perm(h, 0, 0x2222) & MASK;
    hi16.y = __byte_perm(g, 0, 0x2222) & MASK;
    hi16.z = __byte_perm(h, 0, 0x3333) & MASK;
    hi16.w = __byte_perm(g, 0, 0x3333) & MASK;
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

// KHW_T: taps known at compile time (9, 1) or 0 for any tap count up to kTcMaxTaps
// KWC:   32-channel words per pipeline step (TcArgs::KWc);  RA: patch rows per expanding thread (1 .. kTcMaxARows)
template <int KHW_T, int KWC, int RA>
__global__ void __launch_bounds__(kTcThreads, 1)
sc_conv_tc_kernel(TcArgs a, const uint32_t *__restrict__ Ab, const uint32_t *__restrict__ Wb,
                  int16_t *__restrict__ out_pos, int16_t *__restrict__ out_neg, int *__restrict__ status, int gate)
{
    extern __shared__ __align__(16) uint8_t smem_raw[];
    // One of a pair of launches, of which the expand stage's verdict on the activation borders (status word 1: 0 =
    // the compact planes are valid) picks one: +1 runs on valid compact planes only, -1 on the standard planes that
    // replaced them.  The whole grid takes the same branch, before any barrier or tensor memory exists.
    if (gate != 0 && (gate > 0) == (status[1] != 0)) return;
    uint8_t *smem = smem_raw + ((128u - (saddr(smem_raw) & 127u)) & 127u);
    const int KHW = KHW_T ? KHW_T : a.KHW;
    const uint32_t a_bytes = 2u * (uint32_t)KWC * (uint32_t)a.rows_a * 16u; // [2*KWc columns][rows_a][16]
    const uint32_t b_bytes = (uint32_t)KHW * 2u * (uint32_t)KWC * kTcN * 16u; // [KHW][2*KWc columns][128][16]
    auto a_buf = [&](int buf) { return smem + (uint32_t)buf * a_bytes; };
    auto b_buf = [&](int buf) { return smem + 2 * a_bytes + (uint32_t)buf * b_bytes; };
    uint64_t *bars = reinterpret_cast<uint64_t *>(smem + 2 * a_bytes + 2 * b_bytes);
    uint32_t *tmem_slot = reinterpret_cast<uint32_t *>(bars + 8);

    const int tid = threadIdx.x, lane = tid & 31;
    // the shuffle tells the compiler what it cannot see: the warp index is the same in every lane
    const int warp = __shfl_sync(0xffffffffu, tid >> 5, 0);
    // Persistent CTA: it runs its tiles as ONE pipeline, so a tile's first loads / expansion and its last epilogue /
    // store overlap the neighbouring tiles' MMAs.  Its k-th tile is tile first_tile + k * tile_stride, of which it
    // computes time slots [slot_lo(k), slot_hi(k)): all of them, except in the first and last tile of a balanced run.
    // (The run is needed at tile switches only: it lives in shared memory, not in registers.)
    const TileRun &run = *reinterpret_cast<const TileRun *>(tmem_slot + 2);
    if (tid == 0)
        *reinterpret_cast<TileRun *>(tmem_slot + 2) = tile_run(a.total_tiles, a.slots, a.balanced, (int)blockIdx.x, (int)gridDim.x);
    auto slot_lo = [&](int k) { return k == 0 ? run.slot_first : 0; };
    auto slot_hi = [&](int k) { return k == run.tiles - 1 ? run.slot_last_end : a.slots; };
    auto tile_origin = [&](int k, long long &o0, int &nc) {
        const int L = run.first_tile + k * run.tile_stride;
        nc = L / a.tiles_x;                                  // 64-channel output chunk
        o0 = (long long)(L - nc * a.tiles_x) * kTcM;         // first candidate of the tile
    };

    // mbarriers (index = operand buffer or accumulator buffer):
    //   full[b]   operands of a step are in shared memory           (one arrival per expanding warp)
    //   empty[b]  the MMAs that read operand buffer b have completed  (one commit per issuing warp); after the last
    //             chunk of a slot this also says that the slot's counts are complete in their accumulator buffer
    //   tfree[t]  accumulator buffer t has been folded                (one arrival per expanding warp)
    //   drain     every MMA of an issuing warp has completed          (one commit per issuing warp, at its exit)
    uint64_t *bar_full = bars, *bar_empty = bars + 2, *bar_tfree = bars + 4, *bar_drain = bars + 6;
    if (tid == 0) {
        asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(bar_drain)), "r"(kTcM / kTcSub) : "memory");
        for (int b = 0; b < 2; b++) {
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(&bar_full[b])), "r"(kTcWorkers / 32) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(&bar_empty[b])), "r"(kTcM / kTcSub) : "memory");
            asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(saddr(&bar_tfree[b])), "r"(kTcWorkers / 32) : "memory");
        }
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 0) {
        // two accumulator buffers of 2 row blocks x 128 columns: the whole tensor memory of the SM.  The allocation
        // blocks until all 512 columns are free, so this kernel assumes it is the only user of tensor memory on its
        // SM: its > 113 KB of dynamic shared memory keeps a second CTA of itself away, but a kernel of ANOTHER stream
        // that holds tensor memory (the FXP conv of this library, a vendor GEMM) would make the allocation wait for
        // that kernel's CTA to finish.  Callers that overlap streams must serialise this kernel with such kernels.
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(saddr(tmem_slot)),
                     "r"(512u) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;
    const int my_tiles = run.tiles;

    // instruction descriptor: int32 accumulators, signed int8 operands, both K-major, N = 128, M = 128
    const uint32_t idesc = (2u << 4) | (1u << 7) | (1u << 10) | ((uint32_t)(kTcN >> 3) << 17) | ((uint32_t)(kTcSub >> 4) << 24);
    const uint32_t a_lbo = (uint32_t)a.rows_a * 16, b_lbo = kTcN * 16;
    const int wrow_words = KHW * a.CW;                 // weight words per row and slot

    // running sums: this thread owns row block (warp/4)%2, TMEM lane 32*(warp%4)+lane and 64 columns (warp/8 = 0:
    // positive block, 1: negative block), two 16-bit sums per register as the packed TMEM load delivers them
    uint32_t acc[32];
#pragma unroll
    for (int j = 0; j < 32; j++) acc[j] = 0u;
    const uint32_t my_tcol = ((uint32_t)((warp & 3) * 32) << 16) + (uint32_t)(((warp >> 2) & 1) * kTcN + (warp >> 3) * 64);
    const uint32_t n2 = ((uint32_t)a.n_or << kTcScaleLog2) * 0x00010001u; // the clamp, in accumulator units, twice

    // ---- what an expanding thread loads and writes -------------------------------------------------------------
    // Bit words of a step are fetched into registers two steps before their MMAs so that L2 latency is hidden; the
    // loads walk the steps in order, so the step-dependent part of every address is a running pointer.
    //   weights: item e = tid + 512*i, row = e & 127, (tap, word) = e >> 7  -> wbits[i]
    //   patch:   row g = tid + 512*r of the residue planes                  -> abits[r][word]
    // weight words per thread and step: ceil(taps * words / 4) when the tap count is known at compile time
    constexpr int kMyB = KHW_T ? (KHW_T * KWC + 3) / 4 : kTcMaxBWords;
    uint32_t wbits[kMyB], abits[RA][KWC];
    const int w_row = tid & (kTcN - 1), w_rest0 = tid >> 7;               // (tap, word) index of item 0
    const int w_half = KWC == 2 ? (w_rest0 & 1) : 0;
    const int w_tap0 = KWC == 2 ? (w_rest0 >> 1) : w_rest0;
    const int w_items = KHW * KWC;                                      // (tap, word) pairs per step
    const size_t w_item_stride = (size_t)(4 / KWC) * a.CW * kTcN;       // item i -> i + 1: 4 pairs further
    const uint32_t *w_ptr = Wb, *a_plane = Ab, *pf_plane = Ab;
    uint32_t a_off[RA]; // stored-grid position of the thread's patch rows, ~0u: outside the tensor
    const bool pf_on = (a.CW % KWC) == 0;                                // planes are then visited in storage order
    int ld_ck = 0, ld_left = 0, ld_tile = -1;
    // point the loads at tile k of this CTA: slot 0, chunk 0
    auto load_tile = [&](int k) {
        long long o0;
        int nc;
        tile_origin(k, o0, nc);
        const int slot0 = slot_lo(k);                                      // first slot of the tile
        ld_tile = k;
        ld_ck = 0;
        ld_left = (slot_hi(k) - slot0) * a.CK;
        w_ptr = Wb + ((size_t)nc * a.slots + slot0) * kTcN * wrow_words + ((size_t)w_tap0 * a.CW + w_half) * kTcN + w_row;
        a_plane = Ab + (size_t)slot0 * a.CW * a.NHWp;                       // bit plane of the first slot, word 0
        pf_plane = a_plane + (size_t)kTcPrefetch * KWC * a.NHWp;
#pragma unroll
        for (int r = 0; r < RA; r++) {
            const int g = tid + kTcWorkers * r;
            a_off[r] = ~0u;
            if (g < a.rows_a) {
                const int plane = g / a.Mh, q = g - plane * a.Mh;
                // candidate indices fit 31 bits (checked on the host); rows before the first stored pixel wrap around
                // to large values and are zero like the rows behind the last one
                const uint32_t o = (uint32_t)o0 + (uint32_t)q - (uint32_t)a.shift;
                if (o < (uint32_t)a.total_o) {
                    const uint32_t t = o / (uint32_t)a.Wo, j = o - t * (uint32_t)a.Wo;
                    const uint32_t n = t / (uint32_t)a.Ho, i = t - n * (uint32_t)a.Ho;
                    const int rh = plane / a.nrw, rw = plane - rh * a.nrw;
                    a_off[r] = (n * (uint32_t)a.Hrows + i * (uint32_t)a.nrh + (uint32_t)rh) * (uint32_t)a.Wrow +
                               (uint32_t)(rw * a.Wq) + j; // < NHWp < 2^32
                }
            }
        }
    };
    auto load_bits = [&]() {
        const int words_left = a.CW - ld_ck * KWC; // words of this chunk that exist
#pragma unroll
        for (int i = 0; i < kMyB; i++) {
            const bool ok = w_rest0 + 4 * i < w_items && w_half < words_left;
            wbits[i] = ok ? __ldg(w_ptr + i * w_item_stride) : 0u;
        }
#pragma unroll
        for (int r = 0; r < RA; r++) {
            abits[r][0] = a_off[r] != ~0u ? __ldg(a_plane + a_off[r]) : 0u;
            if (KWC == 2) abits[r][KWC - 1] = (a_off[r] != ~0u && words_left > 1) ? __ldg(a_plane + a.NHWp + a_off[r]) : 0u;
        }
        // the patch bits stream from HBM: pull the lines of a later step into L2 (one lane per 128-byte line)
        if (pf_on && lane == 0 && ld_left > kTcPrefetch) {
#pragma unroll
            for (int r = 0; r < RA; r++)
                if (a_off[r] != ~0u) {
                    asm volatile("prefetch.global.L2 [%0];" ::"l"(pf_plane + a_off[r]));
                    if (KWC == 2) asm volatile("prefetch.global.L2 [%0];" ::"l"(pf_plane + a.NHWp + a_off[r]));
                }
        }
        // advance to the next step: next chunk of the slot, or chunk 0 of the next slot
        ld_left--;
        if (++ld_ck == a.CK) {
            ld_ck = 0;
            w_ptr += ((size_t)wrow_words - (size_t)KWC * (a.CK - 1)) * kTcN;
            a_plane += (size_t)(a.CW - KWC * (a.CK - 1)) * a.NHWp;
        } else {
            w_ptr += (size_t)KWC * kTcN;
            a_plane += (size_t)KWC * a.NHWp;
        }
        pf_plane += (size_t)KWC * a.NHWp;
        if (ld_left == 0 && ld_tile + 1 < my_tiles) load_tile(ld_tile + 1); // the next call fetches the next tile
    };
    // per-thread shared-memory offsets of the expansion targets (buffer 0)
    const uint32_t b_dst0 = (uint32_t)(((w_tap0 * 2 * KWC + 2 * w_half) * kTcN + w_row) * 16);
    const uint32_t a_kcol = (uint32_t)a.rows_a * 16;
    auto expand_bits = [&](int buf) {
        uint8_t *b_s = b_buf(buf) + b_dst0, *a_s = a_buf(buf) + (uint32_t)tid * 16;
#pragma unroll
        for (int i = 0; i < kMyB; i++) {
            if (w_rest0 + 4 * i < w_items) {
                uint8_t *dst = b_s + i * (8 * kTcN * 16); // 4 (tap, word) pairs = 8 K-columns further
                uint4 lo16, hi16;
                spread32<kTcMaskW>(wbits[i], lo16, hi16);
                *reinterpret_cast<uint4 *>(dst) = lo16;
                *reinterpret_cast<uint4 *>(dst + kTcN * 16) = hi16;
            }
        }
#pragma unroll
        for (int r = 0; r < RA; r++) {
            if (tid + kTcWorkers * r < a.rows_a) {
                uint8_t *dst = a_s + r * (kTcWorkers * 16);
                uint4 lo16, hi16;
                spread32<kTcMaskA>(abits[r][0], lo16, hi16);
                *reinterpret_cast<uint4 *>(dst) = lo16;
                *reinterpret_cast<uint4 *>(dst + a_kcol) = hi16;
                if (KWC == 2) {
                    spread32<kTcMaskA>(abits[r][KWC - 1], lo16, hi16);
                    *reinterpret_cast<uint4 *>(dst + 2 * a_kcol) = lo16;
                    *reinterpret_cast<uint4 *>(dst + 3 * a_kcol) = hi16;
                }
            }
        }
    };
    // count -> min(count, n) -> running sums, for the slot whose accumulators sit in TMEM buffer `tbuf`
    auto slot_epilogue = [&](int tbuf) {
        const uint32_t taddr = tmem_base + my_tcol + (uint32_t)(tbuf * 2 * kTcN);
        uint32_t v0[16], v1[16];
        REXSC_TMEM_LD16_PACKED(v0, taddr);
        REXSC_TMEM_LD16_PACKED(v1, taddr + 32u);
        asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
        if (!a.descale_each) {
#pragma unroll
            for (int j = 0; j < 16; j++) {
                acc[j] += __vminu2(v0[j], n2);
                acc[16 + j] += __vminu2(v1[j], n2);
            }
        } else {
#pragma unroll
            for (int j = 0; j < 16; j++) {
                acc[j] += (__vminu2(v0[j], n2) >> kTcScaleLog2) & kDescaleMask;
                acc[16 + j] += (__vminu2(v1[j], n2) >> kTcScaleLog2) & kDescaleMask;
            }
        }
        asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    };
    // One thread issues the MMAs of one 128-row block.  A single thread gets one 128-column MMA through about every
    // 128 clocks, half of what the tensor core can take, so the two row blocks are issued from two warps.  The
    // issuing warps share their schedulers with the expanding warps, so the loop is kept to a few instructions per
    // MMA: fully unrolled over taps, per-tap operand offsets in registers, descriptors patched in their low word
    // (the start-address field counts 16-byte units, i.e. operand rows, from bit 0; no carry leaves the field
    // because shared memory ends below 256 KB).
    const int my_sub = warp - kTcWorkers / 32;
    uint32_t a_tap[kTcMaxTaps];
#pragma unroll
    for (int tap = 0; tap < kTcMaxTaps; tap++)
        a_tap[tap] = (my_sub >= 0 && tap < KHW) ? (uint32_t)(my_sub * kTcSub + a.tap_off[tap]) : 0u;
    const uint64_t da_proto = desc_interleaved(saddr(a_buf(0)), a_lbo), db_proto = desc_interleaved(saddr(b_buf(0)), b_lbo);
    const uint32_t da_hi = (uint32_t)(da_proto >> 32), db_hi = (uint32_t)(db_proto >> 32);
    const uint32_t a_kk = 2u * (uint32_t)a.rows_a;             // rows between the 32-channel words of a chunk
    const uint32_t b_tap = 2u * (uint32_t)KWC * kTcN;        // rows between taps of the weight operand
    auto issue_mmas = [&](int step, int s, int ck) {
        const int buf = step & 1;
        const uint32_t da_lo = (uint32_t)da_proto + (uint32_t)buf * (a_bytes >> 4);
        const uint32_t db_lo = (uint32_t)db_proto + (uint32_t)buf * (b_bytes >> 4);
        const uint32_t d_addr = tmem_base + (uint32_t)((s & 1) * 2 * kTcN + my_sub * kTcN);
        const bool two = KWC == 2 && ck * 2 + 1 < a.CW; // a second 32-channel word in this chunk
        const uint32_t first_acc = ck > 0 ? 1u : 0u;
#pragma unroll
        for (int tap = 0; tap < (KHW_T ? KHW_T : kTcMaxTaps); tap++) {
            if (KHW_T || tap < a.KHW) {
#pragma unroll
                for (int kk = 0; kk < 2; kk++) {
                    if (kk == 1 && !two) break;
                    const uint32_t alo = da_lo + a_tap[tap] + (kk ? a_kk : 0u);
                    const uint32_t blo = db_lo + (uint32_t)tap * b_tap + (uint32_t)(2 * kk * kTcN);
                    const uint32_t accumulate = (tap > 0 || kk > 0) ? 1u : first_acc;
                    asm volatile(
                        "{\n\t.reg .pred p, e;\n\t.reg .b64 da, db;\n\t"
                        "mov.b64 da, {%1, %2};\n\t"
                        "mov.b64 db, {%3, %4};\n\t"
                        "setp.ne.b32 p, %6, 0;\n\t"
                        "elect.sync _|e, 0xffffffff;\n\t"
                        "@e tcgen05.mma.cta_group::1.kind::i8 [%0], da, db, %5, {%7, %7, %7, %7}, p;\n\t}"
                        ::"r"(d_addr), "r"(alo), "r"(da_hi), "r"(blo), "r"(db_hi), "r"(idesc), "r"(accumulate), "r"(0u)
                        : "memory");
                }
            }
        }
        // the commits arrive on their barriers when every MMA issued so far by this warp has completed
        asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
                     "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(saddr(&bar_empty[buf]))
                     : "memory");
    };

    bool failed = false;
    const int total_steps = run.slots * a.CK; // pipeline steps of this CTA; slots are numbered through all of its tiles
    // The warps run unsynchronised; every dependence is an mbarrier phase.  Phase parities: barrier index b is used
    // by steps (or slots) b, b + 2, ...; its k-th completion has parity k & 1.  A timed-out wait ends the warp's
    // loop; the warps that depend on it time out in turn, so everybody reaches the end of the kernel.
    auto wait_on = [&](uint64_t *bar, int k) {
        const bool ok = tc_wait(saddr(bar), (uint32_t)(k & 1));
        return __all_sync(0xffffffffu, ok) != 0;
    };
    auto warp_arrive = [&](uint64_t *bar) {
        __syncwarp();
        if (lane == 0) asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(saddr(bar)) : "memory");
    };
    // running sums -> int16 outputs of the tile whose last slot has just been folded; a row is one candidate of the
    // origin grid, it is an output pixel iff i < OH and j < OW
    auto store_tile = [&](int k) {
        long long o0;
        int nc;
        tile_origin(k, o0, nc);
        const bool shared_tile = slot_hi(k) - slot_lo(k) < a.slots; // other CTAs hold the tile's other time slots
        if (!a.descale_each) {
#pragma unroll
            for (int j = 0; j < 32; j++) acc[j] = (acc[j] >> kTcScaleLog2) & kDescaleMask;
        }
        const uint32_t o = (uint32_t)o0 + (uint32_t)(((warp >> 2) & 1) * kTcSub + (warp & 3) * 32 + lane);
        if (o < (uint32_t)a.total_o) {
            const uint32_t t = o / (uint32_t)a.Wo, n = t / (uint32_t)a.Ho;
            const int ow = (int)(o - t * (uint32_t)a.Wo), oh = (int)(t - n * (uint32_t)a.Ho);
            if (ow < a.OW && oh < a.OH) {
                const int co0 = nc * kTcCout;
                const size_t ohw = (size_t)a.OH * a.OW;
                const size_t m = ((size_t)n * a.OH + oh) * a.OW + ow;
                int16_t *dst = (warp >> 3) ? out_neg : out_pos;
                if (a.balanced == 2) {
                    // Any layout: EVERY tile of the launch adds its sums into outputs that the host cleared, one
                    // 16-bit value per 32-bit atomic add on the word that holds it (no carry leaves the value's half:
                    // the complete sums fit 16 bits; the word's other half gets + 0).  All accesses to these words are
                    // atomic adds, so neighbours stored by other CTAs cannot be lost.
                    const size_t e0 = a.out_nhwc ? m * a.Co + co0 : ((size_t)n * a.Co + co0) * ohw + (size_t)oh * a.OW + ow;
                    const size_t estep = a.out_nhwc ? 1 : ohw;
#pragma unroll
                    for (int j = 0; j < 64; j++) {
                        const uint32_t v = (acc[j >> 1] >> (16 * (j & 1))) & 0xffffu;
                        if (co0 + j < a.Co && v != 0u) {
                            const uintptr_t addr = reinterpret_cast<uintptr_t>(dst + e0 + (size_t)j * estep);
                            atomicAdd(reinterpret_cast<unsigned int *>(addr & ~(uintptr_t)3), v << ((addr & 2u) * 8u));
                        }
                    }
                } else if (a.out_nhwc) {
                    int16_t *row = dst + m * a.Co + co0;
                    if (shared_tile) {
                        // partial sums of this share of the slots: two int16 per 32-bit add, no carry can cross the
                        // halves because the complete sums fit 16 bits (the host cuts tiles for aligned rows only)
                        unsigned int *row32 = reinterpret_cast<unsigned int *>(row);
#pragma unroll
                        for (int j = 0; j < 32; j++) atomicAdd(row32 + j, acc[j]);
                    } else if (a.out_vec && (a.Co & 7) == 0 && co0 + kTcCout <= a.Co) {
#pragma unroll
                        for (int j = 0; j < 32; j += 4)
                            *reinterpret_cast<uint4 *>(row + 2 * j) = make_uint4(acc[j], acc[j + 1], acc[j + 2], acc[j + 3]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 64; j++)
                            if (co0 + j < a.Co) row[j] = (int16_t)((acc[j >> 1] >> (16 * (j & 1))) & 0xffffu);
                    }
                } else {
#pragma unroll
                    for (int j = 0; j < 64; j++)
                        if (co0 + j < a.Co)
                            dst[((size_t)n * a.Co + co0 + j) * ohw + (size_t)oh * a.OW + ow] =
                                (int16_t)((acc[j >> 1] >> (16 * (j & 1))) & 0xffffu);
                }
            }
        }
#pragma unroll
        for (int j = 0; j < 32; j++) acc[j] = 0u;
    };
    if (warp >= kTcWorkers / 32) {
        // ---- MMA-issuing warps: operands ready -> accumulator free -> issue -> commit ----
        int s = 0, ck = 0; // slot (counted through all tiles) and chunk of the step
        for (int step = 0; step < total_steps; step++) {
            if (!wait_on(&bar_full[step & 1], step >> 1)) { failed = true; break; }
            if (ck == 0 && s >= 2 && !wait_on(&bar_tfree[s & 1], (s >> 1) - 1)) { failed = true; break; }
            asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            issue_mmas(step, s, ck);
            if (++ck == a.CK) { ck = 0; s++; }
        }
        // Whatever way the loop ended: arrive on the drain barrier once all MMAs this warp has issued are complete,
        // so that tensor memory is not released under an MMA still in flight after a timed-out wait.
        asm volatile("{\n\t.reg .pred e;\n\telect.sync _|e, 0xffffffff;\n\t"
                     "@e tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];\n\t}" ::"r"(saddr(bar_drain))
                     : "memory");
    } else {
        // ---- expanding / folding warps ----
        load_tile(0);
        load_bits();
        expand_bits(0);
        asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
        warp_arrive(&bar_full[0]);
        if (total_steps > 1) load_bits();
        int s_prev = 0, ck_prev = -1; // slot (counted through all tiles) and chunk of step - 1
        int tile_prev = 0, slots_left_prev = slot_hi(0) - slot_lo(0); // tile of step - 1, its slots still to fold
        for (int step = 0; step <= total_steps; step++) {
            // the previous step's MMAs: its operand buffer is free again and, after the last chunk of a slot, the
            // slot's counts are complete
            if (step > 0) {
                if (!wait_on(&bar_empty[(step - 1) & 1], (step - 1) >> 1)) { failed = true; break; }
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
            if (step + 1 < total_steps) {
                expand_bits((step + 1) & 1);
                asm volatile("fence.proxy.async.shared::cta;" ::: "memory");
                warp_arrive(&bar_full[(step + 1) & 1]);
                if (step + 2 < total_steps) load_bits();
            }
            // fold the slot that the previous step completed and hand its accumulators back
            if (ck_prev == a.CK - 1) {
                slot_epilogue(s_prev & 1);
                warp_arrive(&bar_tfree[s_prev & 1]);
                if (--slots_left_prev == 0) {
                    store_tile(tile_prev);
                    tile_prev++;
                    slots_left_prev = slot_hi(tile_prev) - slot_lo(tile_prev);
                }
            }
            if (++ck_prev == a.CK) { ck_prev = 0; s_prev++; }
        }
    }
    if (failed && lane == 0) atomicExch(status, 4);
    // (a warp whose wait timed out leaves its share of the remaining tiles unwritten; the status word reports it)

    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 0) {
        // bounded like every other wait; in a run without time-outs the MMAs are long complete and this returns at once
        if (!wait_on(bar_drain, 0) && lane == 0) atomicExch(status, 4);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(512u) : "memory");
    }
}

// Tensor-pipe issue-rate probe: back-to-back int8 MMAs (M128 x N x K32) on fixed shared-memory operands.
// Zeroes the output rows of every tile that two CTAs of a balanced launch share (see TcArgs::balanced).  Block b looks
// at the cut between runs b and b + 1; a cut inside a tile makes that tile shared.  `grid` is the conv launch's grid.
__global__ void __launch_bounds__(kTcM)
zero_shared_tiles_kernel(TcArgs a, int grid, int16_t *__restrict__ out_pos, int16_t *__restrict__ out_neg,
                         const int *__restrict__ status, int gate)
{
    if (gate != 0 && (gate > 0) == (status[1] != 0)) return;
    const long long units = (long long)a.total_tiles * a.slots;
    const long long cut = units * ((int)blockIdx.x + 1) / grid;
    if (cut % a.slots == 0) return;
    const int L = (int)(cut / a.slots), nc = L / a.tiles_x;
    const uint32_t o0 = (uint32_t)(L - nc * a.tiles_x) * kTcM;
    // One row (candidate) per thread decodes its output position; then the warp writes its 32 rows one after the other,
    // lane l the l-th of the row's 32 words of each sign (rows are 4-byte aligned and hold whole 64-channel chunks, or
    // the host would not have cut tiles).
    const int lane = threadIdx.x & 31;
    const uint32_t o = o0 + threadIdx.x; // blockDim.x == kTcM
    long long word0 = -1;                // first 32-bit word of the row, -1: the candidate is no output pixel
    if (o < (uint32_t)a.total_o) {
        const uint32_t t = o / (uint32_t)a.Wo, n = t / (uint32_t)a.Ho;
        const int ow = (int)(o - t * (uint32_t)a.Wo), oh = (int)(t - n * (uint32_t)a.Ho);
        if (ow < a.OW && oh < a.OH)
            word0 = (long long)(((((size_t)n * a.OH + oh) * a.OW + ow) * a.Co + (size_t)nc * kTcCout) / 2);
    }
    uint32_t *pos32 = reinterpret_cast<uint32_t *>(out_pos), *neg32 = reinterpret_cast<uint32_t *>(out_neg);
#pragma unroll 4
    for (int j = 0; j < 32; j++) {
        const long long w = __shfl_sync(0xffffffffu, word0, j);
        if (w >= 0) {
            pos32[w + lane] = 0u;
            neg32[w + lane] = 0u;
        }
    }
}

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

// geometry of the tensor-core kernel for one plan; ok = false when the layer does not fit
struct TcGeom {
    bool ok;
    int planes, Ho, Wo, Mh, rows_a, KWc, CK, CW;
    size_t smem;
    int tap_off[kTcMaxTaps];
};

TcGeom tc_geometry(const ConvPlan &p)
{
    TcGeom g{};
    g.ok = false;
    if (p.KHW > kTcMaxTaps || p.KHW < 1) return g;
    g.planes = p.nrh * p.nrw;
    g.Ho = p.Hrows / p.nrh;
    g.Wo = p.Wq;
    int max_shift = 0;
    for (int kh = 0; kh < p.KH; kh++)
        for (int kw = 0; kw < p.KW; kw++) {
            const int shift = (kh / p.sh) * g.Wo + kw / p.sw;
            if (shift > max_shift) max_shift = shift;
        }
    g.Mh = (kTcM + max_shift + 7) / 8 * 8;
    g.rows_a = g.planes * g.Mh;
    if (g.rows_a > kTcMaxARows * kTcWorkers) return g;
    for (int t = 0; t < kTcMaxTaps; t++) g.tap_off[t] = 0;
    for (int kh = 0; kh < p.KH; kh++)
        for (int kw = 0; kw < p.KW; kw++) {
            const int plane = (kh % p.sh) * p.nrw + kw % p.sw; // residues below nrh / nrw by construction of the grid
            g.tap_off[kh * p.KW + kw] = plane * g.Mh + (kh / p.sh) * g.Wo + kw / p.sw;
        }
    g.CW = (p.C + 31) / 32;
    for (int kwc = g.CW >= 2 ? 2 : 1; kwc >= 1; kwc--) {
        const size_t need = 2 * ((size_t)2 * kwc * g.rows_a * 16 + (size_t)p.KHW * 2 * kwc * kTcN * 16) + 8 * 8 + 8 + sizeof(TileRun) + 128;
        if (need <= 227 * 1024 && p.KHW * kwc <= 4 * kTcMaxBWords) {
            g.KWc = kwc;
            g.CK = (g.CW + kwc - 1) / kwc;
            // the kernel owns the SM's whole tensor memory: ask for enough shared memory that no second CTA is co-scheduled
            g.smem = need > 120 * 1024 ? need : 120 * 1024;
            g.ok = true;
            break;
        }
    }
    return g;
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
    if (p.Hrows % p.nrh != 0) return false;
    const TcGeom g = tc_geometry(p);
    if (!g.ok) return false;
    const long long cap = p.n_or < p.Kdot ? p.n_or : p.Kdot;                   // largest per-slot contribution
    if ((long long)p.words * 32 * cap > 65535) return false;                  // 16-bit running sums
    if (((long long)p.Kdot << kTcScaleLog2) > 65535) return false;            // 16-bit packed accumulator reads
    if (p.Kdot > (1 << 24)) return false;
    const long long total_o = (long long)p.N * g.Ho * g.Wo;
    if (total_o + kTcM > 0x7fffffffLL) return false;                          // 31-bit candidate indices
    if ((total_o + kTcM - 1) / kTcM * ((p.Co + kTcCout - 1) / kTcCout) > 0x7fffffffLL) return false; // tile index: int
    if (p.NHWp > 0xfffffffeLL) return false;                                  // 32-bit position offsets
    return true;
}

size_t conv_tc_workspace_bytes(const ConvPlan &p)
{
    const int CW = (p.C + 31) / 32, NC = (p.Co + kTcCout - 1) / kTcCout;
    const size_t ab = (size_t)p.words * 32 * CW * p.NHWp * 4;
    const size_t wb = (size_t)NC * p.words * 32 * kTcN * p.KHW * CW * 4;
    return align_up(ab, 256) + align_up(wb, 256);
}

// byte offset of the weight bit planes Wb inside the tensor-core region of the workspace (Ab comes first)
size_t conv_tc_weight_offset(const ConvPlan &p)
{
    const int CW = (p.C + 31) / 32;
    return align_up((size_t)p.words * 32 * CW * p.NHWp * 4, 256);
}

static int device_sms(int *sms)
{
    int dev = 0;
    REXSC_CUDA_CHECK(cudaGetDevice(&dev));
    REXSC_CUDA_CHECK(cudaDeviceGetAttribute(sms, cudaDevAttrMultiProcessorCount, dev));
    return REXSC_OK;
}

int launch_conv_tc(const ConvPlan &p, const rexsc_sc_conv_desc &d, void *d_tc_ws, size_t weight_offset, int16_t *d_pos,
                   int16_t *d_neg, int *d_status, int gate, cudaStream_t st)
{
    if (!conv_tc_supported(p)) return REXSC_E_UNSUPPORTED;
    const TcGeom g = tc_geometry(p);
    const int CW = g.CW, NC = (p.Co + kTcCout - 1) / kTcCout;
    const int slots = p.words * 32;
    const uint32_t *Ab = static_cast<const uint32_t *>(d_tc_ws);
    const uint32_t *Wb = reinterpret_cast<const uint32_t *>(static_cast<const uint8_t *>(d_tc_ws) + weight_offset);
    TcArgs a;
    a.OH = p.OH; a.OW = p.OW; a.KHW = p.KHW; a.Co = p.Co;
    a.CW = CW; a.KWc = g.KWc; a.CK = g.CK;
    a.nrh = p.nrh; a.nrw = p.nrw; a.Wq = p.Wq; a.Hrows = p.Hrows; a.Wrow = p.Wrow;
    a.Ho = g.Ho; a.Wo = g.Wo; a.Mh = g.Mh; a.rows_a = g.rows_a;
    a.shift = p.origin ? g.Wo + 1 : 0;
    a.slots = slots;
    a.total_o = (long long)p.N * g.Ho * g.Wo;
    a.tiles_x = (int)((a.total_o + kTcM - 1) / kTcM);
    int sms = 0;
    if (int rc = device_sms(&sms)) return rc;
    a.total_tiles = a.tiles_x * NC;
    // One persistent CTA per SM (the kernel owns the SM's tensor memory).  Whole tiles dealt round-robin leave SMs idle
    // in the last wave (900 tiles on 148 SMs: 7 waves for the work of 6.1); cutting the (tile, slot) sequence into
    // equal runs does not.  The cut tiles are summed with packed 32-bit atomic adds, which need 4-byte aligned rows
    // of whole 64-channel chunks; the fallback launch of a gated pair keeps whole tiles (it is the rare one and a
    // second clearing kernel would cost every call).
    const long long units = (long long)a.total_tiles * slots;
    const bool aligned4 = ((reinterpret_cast<uintptr_t>(d_pos) | reinterpret_cast<uintptr_t>(d_neg)) & 3u) == 0;
    const bool rows_ok = d.out_channels_last && (p.Co % kTcCout) == 0 && aligned4;
    unsigned grid = (unsigned)(a.total_tiles < sms ? a.total_tiles : sms);
    a.balanced = 0;
    static const bool allow_balanced = !(getenv("REXSC_TC_BALANCED") && getenv("REXSC_TC_BALANCED")[0] == '0');
    // (measured: tiles with little tensor work per slot -- 1x1 filters on up to 256 channels -- gain nothing: their
    // time goes to the per-slot hand-offs, and the atomic stores of the cut tiles cost more than the idle SMs did)
    const bool heavy_slots = p.KHW * CW >= 16 || a.total_tiles < sms;
    if (allow_balanced && heavy_slots && rows_ok && gate >= 0 && a.total_tiles % sms != 0) {
        // short layers: as many CTAs as leaves each about 64 pipeline steps to amortise its prologue
        long long ctas = units * g.CK / 64;
        if (ctas < 1) ctas = 1;
        if (ctas > sms) ctas = sms;
        const long long waves = (a.total_tiles + sms - 1) / sms;
        // worth a clearing launch when the last wave of whole tiles would waste more than 1 % of the SM time
        if ((double)a.total_tiles / sms < 0.99 * (double)waves || ctas > (long long)grid) {
            a.balanced = 1;
            grid = (unsigned)ctas;
        }
    }
    // Outputs without such rows (NCHW, a ragged last chunk): clear them whole and let every tile add single 16-bit
    // values -- affordable while the outputs are small, which is where whole tiles waste most (deep layers with few
    // tiles per SM).  The element count must be even so that the last value's 32-bit word ends inside the tensor.
    const size_t out_elems = (size_t)p.M * p.Co;
    if (allow_balanced && heavy_slots && !rows_ok && aligned4 && (out_elems & 1) == 0 && out_elems * sizeof(int16_t) <= ((size_t)16 << 20) &&
        gate >= 0 && a.total_tiles % sms != 0) {
        long long ctas = units * g.CK / 64;
        if (ctas < 1) ctas = 1;
        if (ctas > sms) ctas = sms;
        const long long waves = (a.total_tiles + sms - 1) / sms;
        if ((double)a.total_tiles / sms < 0.95 * (double)waves || ctas > (long long)grid) {
            a.balanced = 2;
            grid = (unsigned)ctas;
            REXSC_CUDA_CHECK(cudaMemsetAsync(d_pos, 0, out_elems * sizeof(int16_t), st));
            REXSC_CUDA_CHECK(cudaMemsetAsync(d_neg, 0, out_elems * sizeof(int16_t), st));
        }
    }
    if (a.balanced == 1 && grid > 1) {
        zero_shared_tiles_kernel<<<grid - 1, kTcM, 0, st>>>(a, (int)grid, d_pos, d_neg, d_status, gate);
        REXSC_LAUNCH_CHECK("zero_shared_tiles_kernel");
    }
    a.NHWp = p.NHWp; a.out_nhwc = d.out_channels_last;
    if ((reinterpret_cast<uintptr_t>(d_pos) | reinterpret_cast<uintptr_t>(d_neg)) & 1u) return REXSC_E_BAD_ARG;
    a.out_vec = ((reinterpret_cast<uintptr_t>(d_pos) | reinterpret_cast<uintptr_t>(d_neg)) & 15u) == 0 ? 1 : 0;
    {
        const long long cap = p.n_or < p.Kdot ? p.n_or : p.Kdot;
        a.descale_each = (((long long)slots * cap) << kTcScaleLog2) > 65535 ? 1 : 0;
        a.n_or = (int)cap; // a count never exceeds the dot length, so clamping there changes nothing
    }
    for (int t = 0; t < kTcMaxTaps; t++) a.tap_off[t] = g.tap_off[t];
    const int ra = (g.rows_a + kTcWorkers - 1) / kTcWorkers;
    auto pick = [&](auto khw_tag) {
        constexpr int KHW_T = decltype(khw_tag)::value;
        if (g.KWc == 2) return ra == 1 ? sc_conv_tc_kernel<KHW_T, 2, 1> : sc_conv_tc_kernel<KHW_T, 2, kTcMaxARows>;
        return ra == 1 ? sc_conv_tc_kernel<KHW_T, 1, 1> : sc_conv_tc_kernel<KHW_T, 1, kTcMaxARows>;
    };
    auto kernel = p.KHW == 9 ? pick(std::integral_constant<int, 9>{})
                : p.KHW == 1 ? pick(std::integral_constant<int, 1>{}) : pick(std::integral_constant<int, 0>{});
    REXSC_CUDA_CHECK(cudaFuncSetAttribute(kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)g.smem));
    kernel<<<grid, kTcThreads, g.smem, st>>>(a, Ab, Wb, d_pos, d_neg, d_status, gate);
    REXSC_LAUNCH_CHECK("sc_conv_tc_kernel");
    return REXSC_OK;
}

} // namespace rexsc
