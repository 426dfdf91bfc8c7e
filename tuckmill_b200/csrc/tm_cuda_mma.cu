// Prefill GEMM on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
// Contract (the reference's matrix-unit GEMM, native/metal/kernels.metal:503-635
// and native/metal/tm_metal.h:168-189): Y[b, :] = W X[b, :] for b < batch, X at
// f32 offset x_off, Y at y_off, tolerance-qualified.  The reference multiplies
// f32 operands on 8x8 SIMD-group tiles; this kernel follows the declared f16
// operand profile instead: x and d*q are rounded to binary16 (each once, to
// nearest even), products accumulate in f32 in tensor memory.
//
// Persistent kernel, one CTA per SM, tiles of 128 (weight rows) x 2*BN (tokens)
// of Y^T handed out round-robin.  Three facts measured on this part shape it:
//  * the thread that issues tcgen05.mma cannot hide its own barrier waits and
//    commits behind a K step of four MMAs, so TWO threads issue, each into its
//    own BN-column accumulator (two token sub-tiles against the same weight
//    rows): while one waits, the other's MMAs keep the tensor pipe busy;
//  * staging both operands in shared memory saturates the shared-memory data
//    path before the tensor pipe, so the dequantised weight tile is the MMA's A
//    operand IN TENSOR MEMORY and never touches shared memory;
//  * a weight tile converted once now serves 2*BN tokens.
// Tensor memory: two BN-column accumulators + (512 - 2*BN)/32 A stages of 32 columns.
// Roles by warp:
//   0-7    converters: warps q and q+4 own tensor-memory lanes 32q..32q+31 and
//          take alternate K steps; a thread reads its row's 64 raw bytes (TMA,
//          64-byte swizzle), turns them into f16 d*q (byte permute into 1024+u,
//          subtract 1152, multiply by d) and writes them with tcgen05.st; block
//          scales come straight from global memory, several K steps ahead
//   8-15   epilogue: tensor memory -> registers -> Y; four warps (one lane quarter each) per accumulator
//   16     one thread issues the TMA loads of the raw weight tile
//   17     one thread issues the TMA loads of the two token sub-tiles (f16 copy of X)
//   18,19  one thread each issues tcgen05.mma for its sub-tile; warp 18 allocates tensor memory
// The accumulators are single-buffered (tensor memory is full), so a tile's epilogue is not hidden
// behind the next tile's MMAs: eight warps keep it short.
// Stages are handed over with mbarriers; every wait is bounded and raises an
// abort flag instead of spinning forever.
#include <cuda.h>

#include "tm_cuda_internal.cuh"
#include "tm_cuda_device.cuh"
#include "tm_cuda_symm.cuh"

namespace {

constexpr int kBM = 128;        // weight rows per tile (UMMA M)
constexpr int kBK = 64;         // K per stage: 64 f16 = one 128-byte swizzle row
constexpr int kRawStages = 4;   // raw int8 weight tiles in flight (8 KB each)
constexpr int kConvWarps = 8, kIssuers = 2, kEpiWarps = 4;
constexpr int kWarpRaw = kConvWarps + kEpiWarps, kWarpTok = kWarpRaw + 1, kWarpMma = kWarpRaw + 2;
constexpr int kMmaThreads = (kWarpMma + kIssuers) * 32;
constexpr int kScaleAhead = 4;  // a converter's own steps (every other K step) between a scale's load and its use
constexpr uint32_t kSpinLimit = 1u << 20;  // a healthy wait is microseconds; this is ~seconds
// Split-K: when it shortens the longest CTA's run (few output tiles on many SMs: a decode batch, a narrow
// projection, a last round that leaves most SMs idle) the K range of every tile is cut into `ksplit`
// equal parts, each its own tile of the persistent grid;
// the parts' accumulators meet in a workspace slot per (tile, part) and the warp that arrives last for a
// (tile, row quarter) adds them IN PART ORDER and runs the epilogue -- no waiting, and a sum that does not
// depend on which part finished last.
// The workspace holds 148 slots of the widest split tile (128 rows x 256 tokens); narrower tiles pack
// more (output tile, part) slots into the same bytes.  Arrival counters: 4 row quarters per output tile.
constexpr uint32_t kSplitSlots = 148;
constexpr uint32_t kSplitSlotFloats = 128u * 256u;
constexpr size_t kSplitCountBytes = 4096;                   // up to 256 output tiles x 4 x u32
constexpr size_t kSplitBytes = (size_t)kSplitSlots * kSplitSlotFloats * 4 + kSplitCountBytes;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

__device__ __forceinline__ void mbar_init(uint64_t *bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(smem_u32(bar)), "r"(count));
}
__device__ __forceinline__ void mbar_arrive(uint64_t *bar) {
    asm volatile("mbarrier.arrive.shared::cta.b64 _, [%0];" ::"r"(smem_u32(bar)) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint64_t *bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(smem_u32(bar)), "r"(bytes) : "memory");
}
// Bounded wait on a phase parity; false (and the abort flag set) when it gives up.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *abort_flag) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < kSpinLimit; ++spin) {
        uint32_t done;
        asm volatile(
            "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.b32 %0, 1, 0, p;\n}\n"
            : "=r"(done)
            : "r"(addr), "r"(parity)
            : "memory");
        if (done) return true;
        if ((spin & 1023u) == 1023u && *abort_flag) return false;
    }
    *abort_flag = 1u;
    return false;
}

// Shared-memory matrix descriptor, K-major operand in the 128-byte swizzle:
// rows are 128 bytes apart, groups of 8 rows 1024 bytes apart (SBO), 16-byte
// chunk c of row r sits at chunk position c ^ (r & 7).
__device__ __forceinline__ uint64_t umma_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFFu) >> 4);       // start address
    d |= (uint64_t)1 << 16;                             // leading byte offset (unused for swizzled K-major)
    d |= (uint64_t)(1024u >> 4) << 32;                  // stride byte offset: 8 rows * 128 B
    d |= (uint64_t)1 << 46;                             // descriptor version (sm_100)
    d |= (uint64_t)2 << 61;                             // layout: SWIZZLE_128B
    return d;
}

// Instruction descriptor, kind::f16: f16 x f16 -> f32, both operands K-major.
__host__ __device__ constexpr uint32_t umma_idesc(uint32_t m, uint32_t n) {
    return (1u << 4) | ((n >> 3) << 17) | ((m >> 4) << 24);
}

// D[tmem] (+)= A[tmem] * B[smem] over one K step of 64: four MMAs of K = 16 in a single block (one
// predicate set-up for all four).  A is 128 lanes x 8 tensor-memory columns per MMA (16 f16 per row, two per column); B advances 32 bytes = 2 descriptor units, in the low word only.
__device__ __forceinline__ void umma_f16_ts_x4(uint32_t d_tmem, uint32_t a_tmem, uint32_t b_lo, uint32_t b_hi,
                                               uint32_t idesc, uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p, q;\n .reg .b64 b0, b1, b2, b3;\n .reg .b32 a1, a2, a3, l1, l2, l3;\n"
        " setp.ne.b32 p, %5, 0;\n setp.eq.b32 q, 0, 0;\n"
        " add.u32 a1, %1, 8;\n add.u32 a2, %1, 16;\n add.u32 a3, %1, 24;\n"
        " add.u32 l1, %2, 2;\n add.u32 l2, %2, 4;\n add.u32 l3, %2, 6;\n"
        " mov.b64 b0, {%2, %3};\n mov.b64 b1, {l1, %3};\n mov.b64 b2, {l2, %3};\n mov.b64 b3, {l3, %3};\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [%1], b0, %4, p;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [a1], b1, %4, q;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [a2], b2, %4, q;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], [a3], b3, %4, q;\n}\n" ::"r"(d_tmem),
        "r"(a_tmem), "r"(b_lo), "r"(b_hi), "r"(idesc), "r"(accumulate)
        : "memory");
}
__device__ __forceinline__ void umma_commit(uint64_t *bar) {
    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(smem_u32(bar))
                 : "memory");
}
__device__ __forceinline__ void tma_load_2d(void *dst, const CUtensorMap *map, int x, int y, uint64_t *bar) {
    asm volatile(
        "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
            smem_u32(dst)),
        "l"(map), "r"(smem_u32(bar)), "r"(x), "r"(y)
        : "memory");
}

// Eight quants (two 32-bit words) -> eight f16 values d*q, as four half2 words.
__device__ __forceinline__ void dequant8(uint32_t w0, uint32_t w1, __half2 d2, uint32_t *out) {
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480));  // 1152.0
    const uint32_t u0 = w0 ^ 0x80808080u, u1 = w1 ^ 0x80808080u;  // q + 128 as unsigned bytes
    // byte b of u -> f16 bits 0x6400 | b == 1024 + b, two lanes per permute
    const uint32_t h[4] = {__byte_perm(u0, 0x64646464u, 0x4140), __byte_perm(u0, 0x64646464u, 0x4342),
                           __byte_perm(u1, 0x64646464u, 0x4140), __byte_perm(u1, 0x64646464u, 0x4342)};
#pragma unroll
    for (int i = 0; i < 4; ++i) {
        const __half2 qh = __hsub2(*(const __half2 *)&h[i], bias);  // exact integers -128..127
        const __half2 v = __hmul2(qh, d2);                          // one rounding: RN(d * q)
        out[i] = *(const uint32_t *)&v;
    }
}

struct mma_args {
    const __half *d;       // [rows][cols/32] block scales
    // The rows may be cut into up to three consecutive parts (q | k | v, gate | up), each with its own
    // dense output Y_p[t * part_rows + r]; every part but the last is a multiple of 128 rows, so a
    // tile never straddles two parts.
    float *y[3];
    uint32_t part_end[3];  // exclusive row bound of each part (the last one is `rows`)
    uint32_t accumulate;   // 1: Y += W X (the residual add folded into the epilogue)
    uint32_t ksplit;       // K parts per output tile (1: none)
    float *kpart;          // [slot][token][128 rows] partial accumulators, slot = output tile * ksplit + part
    uint32_t kslot;        // floats per slot: 128 rows x the tokens of a tile (rounded up to 32)
    uint32_t *kcount;      // [output tile][4 row quarters] arrivals (left at zero)
    // Row split: the epilogue stores this rank's rows straight into EVERY rank's gathered
    // Y[t][rank * rows + r] (peer memory, plain stores over NVLink), so the all-gather overlaps the
    // MMAs of later tiles; the last CTA ends the exchange (tm_symm_finish).  push_world = 0: off.
    float *const *peer;
    uint32_t push_world, push_rank, push_off, push_tail;
    uint32_t rows, cols, batch;
    uint32_t *abort_flag;  // set when a bounded wait gave up
};

// Ring bookkeeping over a running step count g: stage g % D, the consumer waits
// for fill number g / D (parity of it), the producer for drain number g / D - 1.
template <int D>
struct ring {
    static __device__ __forceinline__ uint32_t stage(uint32_t g) { return g % D; }
    static __device__ __forceinline__ uint32_t full_parity(uint32_t g) { return (g / D) & 1u; }
    static __device__ __forceinline__ bool must_wait_empty(uint32_t g) { return g >= (uint32_t)D; }
    static __device__ __forceinline__ uint32_t empty_parity(uint32_t g) { return (g / D - 1u) & 1u; }
};

template <int BN>
struct mma_smem {
    // One ring hands both operands of a K step to the issuers: stage s holds the converted weight tile
    // (tensor-memory columns kACol0 + 32 s) and the token sub-tiles (shared memory), behind ONE full
    // barrier (converter arrivals + the TMA's bytes) and ONE empty barrier (the issuers' commits), so
    // an issuer pays one wait and one commit per step.
    static constexpr int kATmemStages = (512 - kIssuers * BN) / 32;  // what the accumulators leave
    static constexpr int kStages = BN > 128 ? 4 : 6;
    static constexpr uint32_t kRawBytes = kBM * kBK;             // int8
    static constexpr uint32_t kSubBytes = BN * kBK * 2;          // one token sub-tile, f16
    static constexpr uint32_t kBBytes = kIssuers * kSubBytes;    // a stage
    static constexpr uint32_t kBOff = 0;
    static constexpr uint32_t kRawOff = kBOff + kStages * kBBytes;
    static constexpr uint32_t kBarOff = kRawOff + kRawStages * kRawBytes;
    static constexpr uint32_t kBars = 2 * kRawStages + 2 * kStages + kIssuers + 1;
    static constexpr uint32_t kBytes = 1024 + kBarOff + kBars * 8 + 16;
    static constexpr uint32_t kACol0 = kIssuers * BN;  // tensor-memory column of A stage 0, after the accumulators
    static constexpr uint32_t kTmemCols = 512;
    static_assert(kStages % 2 == 0 && kStages <= kATmemStages, "each converter set needs its own A stages");
    static_assert(kBytes <= 232448, "shared memory per CTA");
};

template <int BN>
__global__ void __launch_bounds__(kMmaThreads, 1)
    q8_gemm_mma_kernel(const __grid_constant__ CUtensorMap wmap, const __grid_constant__ CUtensorMap xmap,
                       const mma_args a) {
    using L = mma_smem<BN>;
    constexpr int kStages = L::kStages;
    constexpr uint32_t kTB = kIssuers * BN;  // tokens per tile
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte aligned stage buffers (swizzle atoms), then the barriers.
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    unsigned char *sB = smem + L::kBOff, *sRaw = smem + L::kRawOff;
    uint64_t *raw_full = (uint64_t *)(smem + L::kBarOff), *raw_empty = raw_full + kRawStages;
    uint64_t *full = raw_empty + kRawStages, *empty = full + kStages;
    uint64_t *acc_full = empty + kStages, *acc_empty = acc_full + kIssuers;
    uint32_t *tmem_slot = (uint32_t *)(acc_empty + 1);
    volatile uint32_t *abort_s = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    // A tile of the grid is (output tile, K part): tile / ksplit and tile % ksplit; nkb K steps each.
    const uint32_t ksplit = a.ksplit;
    const uint32_t nkb = (a.cols + kBK - 1) / kBK / ksplit, nb = a.cols / 32u;
    const uint32_t row_tiles = (a.rows + kBM - 1) / kBM, tok_tiles = (a.batch + kTB - 1) / kTB;
    const uint32_t n_tiles = row_tiles * tok_tiles * ksplit;
    // Consecutive tiles share a token tile, so CTAs running side by side read the same X.

    if (tid == 0) {
        for (int s = 0; s < kRawStages; ++s) {
            mbar_init(&raw_full[s], 1);            // the TMA thread's expect_tx arrival
            mbar_init(&raw_empty[s], kConvWarps / 2);  // one arrival per converter warp of the set that read it
        }
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full[s], kConvWarps / 2 + 1);  // the converter set's warps + the TMA thread's expect_tx arrival
            mbar_init(&empty[s], kIssuers);           // one tcgen05.commit per issuer
        }
        for (int s = 0; s < kIssuers; ++s) mbar_init(&acc_full[s], 1);  // tcgen05.commit after a tile's last MMA
        mbar_init(acc_empty, kEpiWarps);                                    // one arrival per epilogue warp
        *abort_s = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == kWarpMma) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"(L::kTmemCols)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    // Programmatic dependent launch: the weight pipeline (TMA of the raw tiles, converters) reads
    // nothing a predecessor writes and starts at once, overlapping the predecessor's tail -- the f16
    // copy of X that precedes every call; the two roles that touch a predecessor's data, the token
    // TMA thread (X) and the epilogue warps (Y), wait for it first.  The successor is let go only
    // by those roles after their wait, so at most this kernel's direct predecessor can still be running.
    if (warp < kConvWarps) {
        // ---------------- converters ----------------
        // Warps q and q + 4 reach tensor-memory lanes 32q..32q+31; set 0 (warps 0-3) converts the even K
        // steps of the running count, set 1 the odd ones.  A thread owns tile row 32q + lane.
        const uint32_t set = (uint32_t)warp >> 2, quarter = (uint32_t)warp & 3u;
        const uint32_t trow = quarter * 32u + (uint32_t)lane;
        const uint32_t rsw = (trow >> 1) & 3u;  // the TMA's 64-byte swizzle: 16-byte piece c of row r sits at c ^ ((r >> 1) & 3)
        const bool pair_load = (nb & 1u) == 0u;  // both scales of a K step in one aligned 4-byte load
        // Scale look-ahead: the position (tile, kb) of this set's step kScaleAhead own-steps in front.
        uint32_t la_tile = blockIdx.x, la_kb = 0;
        auto la_advance = [&](uint32_t n) {
            for (uint32_t i = 0; i < n; ++i)
                if (++la_kb == nkb) {
                    la_kb = 0;
                    la_tile += gridDim.x;
                }
        };
        auto scale_load = [&]() -> uint32_t {
            if (la_tile >= n_tiles) return 0u;
            const uint32_t r = min(((la_tile / ksplit) % row_tiles) * kBM + trow, a.rows - 1u);
            const uint32_t blk = ((la_tile % ksplit) * nkb + la_kb) * 2u;
            const unsigned short *p = (const unsigned short *)a.d + (size_t)r * nb + blk;
            if (pair_load) return __ldg((const uint32_t *)p);
            const uint32_t lo = __ldg(p), hi = blk + 1u < nb ? (uint32_t)__ldg(p + 1) : 0u;
            return lo | (hi << 16);
        };
        la_advance(set);
        // The look-ahead values live in registers with STATIC indices (the loop below is unrolled by
        // the ring length): a rotating copy would read each register right after its load was issued
        // and wait out the whole memory latency every step.
        uint32_t ring_d[kScaleAhead];
#pragma unroll
        for (int i = 0; i < kScaleAhead; ++i) {
            ring_d[i] = scale_load();
            la_advance(2);
        }
        // This set's steps, flat over the CTA's tiles: own step j is running step g = 2j + set.
        const uint32_t my_tiles = blockIdx.x < n_tiles ? (n_tiles - 1u - blockIdx.x) / gridDim.x + 1u : 0u;
        const uint32_t total = my_tiles * nkb, n_own = total > set ? (total - set + 1u) / 2u : 0u;
        bool ok = true;
        for (uint32_t j0 = 0; j0 < n_own && ok; j0 += kScaleAhead) {
#pragma unroll
            for (int u = 0; u < kScaleAhead; ++u) {
                if (j0 + (uint32_t)u >= n_own || !ok) break;
                const uint32_t g = 2u * (j0 + (uint32_t)u) + set;
                const uint32_t sr = ring<kRawStages>::stage(g), sa = ring<kStages>::stage(g);
                // Convert into registers first; the A stage is needed only for the store.
                ok = mbar_wait(&raw_full[sr], ring<kRawStages>::full_parity(g), abort_s);
                const unsigned char *raw = sRaw + sr * L::kRawBytes + trow * kBK;
                const uint32_t dd = ring_d[u];
                const __half2 d_lo = __half2half2(__ushort_as_half((unsigned short)(dd & 0xffffu)));
                const __half2 d_hi = __half2half2(__ushort_as_half((unsigned short)(dd >> 16)));
                // The four 16-byte pieces of this row (k 16c..16c+15) come out of shared memory at once; the
                // raw stage then goes back to the TMA thread, not after the stores below have completed.
                int4 w4[4];
#pragma unroll
                for (uint32_t c = 0; c < 4; ++c) w4[c] = *(const int4 *)(raw + ((c ^ rsw) << 4));
                __syncwarp();
                if (lane == 0) mbar_arrive(&raw_empty[sr]);
                uint32_t v[32];
                dequant8((uint32_t)w4[0].x, (uint32_t)w4[0].y, d_lo, v);
                dequant8((uint32_t)w4[0].z, (uint32_t)w4[0].w, d_lo, v + 4);
                dequant8((uint32_t)w4[1].x, (uint32_t)w4[1].y, d_lo, v + 8);
                dequant8((uint32_t)w4[1].z, (uint32_t)w4[1].w, d_lo, v + 12);
                ring_d[u] = scale_load();
                la_advance(2);
                if (ok && ring<kStages>::must_wait_empty(g))
                    ok = mbar_wait(&empty[sa], ring<kStages>::empty_parity(g), abort_s);
                ok = __all_sync(0xffffffffu, ok);  // the tensor-memory stores below are warp-collective
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                // Register i -> column i of this thread's lane: k = 2i (low half), 2i + 1 (high half).  Two
                // stores of 16 columns: the second half is converted while the first store is in flight.
                const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + L::kACol0 + sa * 32u;
                asm volatile(
                    "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                    "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr),
                    "r"(v[0]), "r"(v[1]), "r"(v[2]), "r"(v[3]), "r"(v[4]), "r"(v[5]), "r"(v[6]), "r"(v[7]), "r"(v[8]),
                    "r"(v[9]), "r"(v[10]), "r"(v[11]), "r"(v[12]), "r"(v[13]), "r"(v[14]), "r"(v[15])
                    : "memory");
                dequant8((uint32_t)w4[2].x, (uint32_t)w4[2].y, d_hi, v + 16);
                dequant8((uint32_t)w4[2].z, (uint32_t)w4[2].w, d_hi, v + 20);
                dequant8((uint32_t)w4[3].x, (uint32_t)w4[3].y, d_hi, v + 24);
                dequant8((uint32_t)w4[3].z, (uint32_t)w4[3].w, d_hi, v + 28);
                asm volatile(
                    "tcgen05.st.sync.aligned.32x32b.x16.b32 [%0], "
                    "{%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16};" ::"r"(taddr + 16u),
                    "r"(v[16]), "r"(v[17]), "r"(v[18]), "r"(v[19]), "r"(v[20]), "r"(v[21]), "r"(v[22]), "r"(v[23]),
                    "r"(v[24]), "r"(v[25]), "r"(v[26]), "r"(v[27]), "r"(v[28]), "r"(v[29]), "r"(v[30]), "r"(v[31])
                    : "memory");
                asm volatile("tcgen05.wait::st.sync.aligned;" ::: "memory");
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(&full[sa]);
            }
        }
    } else if (warp < kWarpRaw) {
        // ---------------- epilogue: tensor memory -> registers -> Y ----------------
        const uint32_t quarter = (uint32_t)warp & 3u;  // a warp reaches tensor-memory lanes 32*(warp%4)..+31
        uint32_t it = 0;
        bool ok = true;
        tmdev::pdl_wait();  // Y (and the split-K slots) belong to the predecessors until they have finished
        tmdev::pdl_trigger();
        for (uint32_t tile = blockIdx.x; tile < n_tiles; tile += gridDim.x, ++it) {
          const uint32_t ot = tile / ksplit, part = tile % ksplit;
          // Split K, pass 0: the accumulators go to this part's workspace slot; pass 1 (only the warp that
          // arrived last for this tile's row quarter): the parts are added in order and stored.
          for (uint32_t pass = 0; pass < (ksplit > 1u ? 2u : 1u) && ok; ++pass) {
          if (pass == 1u) {
              __threadfence();
              __syncwarp();
              uint32_t last = 0u;
              if (lane == 0) last = atomicAdd(a.kcount + ot * 4u + quarter, 1u) == ksplit - 1u ? 1u : 0u;
              last = __shfl_sync(0xffffffffu, last, 0);
              if (!last) break;
              __threadfence();
              if (lane == 0) a.kcount[ot * 4u + quarter] = 0u;  // ready for the next launch
          }
          for (uint32_t sub = 0; sub < (uint32_t)kIssuers && ok; ++sub) {
            const uint32_t tile_row0 = (ot % row_tiles) * kBM;
            const uint32_t rr = tile_row0 + quarter * 32u + (uint32_t)lane;
            const uint32_t tok0 = (ot / row_tiles) * kTB + sub * BN;
            // (selects, not indexing: the arrays are kernel parameters)
            const bool p0 = tile_row0 < a.part_end[0], p1 = tile_row0 < a.part_end[1];
            const uint32_t part_row0 = p0 ? 0u : p1 ? a.part_end[0] : a.part_end[1];
            const uint32_t part_row1 = p0 ? a.part_end[0] : p1 ? a.part_end[1] : a.part_end[2];
            const size_t stride = part_row1 - part_row0;  // rows of this part = token stride of its output
            float *ybase = (p0 ? a.y[0] : p1 ? a.y[1] : a.y[2]) + (rr - part_row0);
            if (pass == 0u) {
                if (ok) ok = mbar_wait(&acc_full[sub], it & 1u, abort_s);
                ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below are warp-collective
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
            }
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                const uint32_t t0 = tok0 + (uint32_t)c0;
                if (t0 >= a.batch) break;  // uniform: the rest of the sub-tile is past the batch
                uint32_t v[32];
                if (pass == 1u) {
                    // this row's 32 tokens of every part, part 0 first
                    const size_t at = ((size_t)(sub * BN + (uint32_t)c0)) * 128u + quarter * 32u + (uint32_t)lane;
#pragma unroll
                    for (int j = 0; j < 32; ++j) v[j] = 0u;
                    for (uint32_t pp = 0; pp < ksplit; ++pp) {
                        const float *src = a.kpart + (size_t)(ot * ksplit + pp) * a.kslot + at;
                        float f[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j) f[j] = __ldcg(src + (size_t)j * 128u);
#pragma unroll
                        for (int j = 0; j < 32; ++j) v[j] = __float_as_uint(pp == 0u ? f[j] : __uint_as_float(v[j]) + f[j]);
                    }
                } else {
                const uint32_t taddr = tmem_base + ((quarter * 32u) << 16) + sub * BN + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,"
                    "%25,%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                      "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
                      "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
                      "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                }
                if (ksplit > 1u && pass == 0u) {
                    float *dst = a.kpart + (size_t)(ot * ksplit + part) * a.kslot +
                                 ((size_t)(sub * BN + (uint32_t)c0)) * 128u + quarter * 32u + (uint32_t)lane;
#pragma unroll
                    for (int j = 0; j < 32; ++j) dst[(size_t)j * 128u] = __uint_as_float(v[j]);
                } else if (rr < a.rows) {
                    // Lane = row: for a fixed token the warp writes 128 contiguous bytes; the addresses
                    // are independent (no add chain between the stores).
                    float *p = ybase + (size_t)t0 * stride;
                    if (a.push_world) {
                        const size_t wide = (size_t)a.push_world * a.rows;  // token stride of the gathered Y
                        const size_t at = a.push_off + (size_t)t0 * wide + (size_t)a.push_rank * a.rows + rr;
                        for (uint32_t pr = 0; pr < a.push_world; ++pr) {
                            float *q = a.peer[pr] + at;
#pragma unroll
                            for (int j = 0; j < 32; ++j)
                                if (t0 + (uint32_t)j < a.batch) q[(size_t)j * wide] = __uint_as_float(v[j]);
                        }
                    } else if (a.accumulate) {
                        // all 32 loads first: a load after a store to the same array cannot be hoisted by
                        // the compiler, and 32 dependent round trips cost more than the tile's main loop
                        float old[32];
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            old[j] = t0 + (uint32_t)j < a.batch ? __ldcg(p + (size_t)j * stride) : 0.0f;
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (t0 + (uint32_t)j < a.batch) p[(size_t)j * stride] = old[j] + __uint_as_float(v[j]);
                    } else if (t0 + 32u <= a.batch) {
#pragma unroll
                        for (int j = 0; j < 32; ++j) p[(size_t)j * stride] = __uint_as_float(v[j]);
                    } else {
#pragma unroll
                        for (int j = 0; j < 32; ++j)
                            if (t0 + (uint32_t)j < a.batch) p[(size_t)j * stride] = __uint_as_float(v[j]);
                    }
                }
            }
          }
            if (!ok) break;
            if (pass == 0u) {
                // The accumulator may be overwritten once every warp has its values in registers.
                asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
                __syncwarp();
                if (lane == 0) mbar_arrive(acc_empty);
            }
          }
            if (!ok) break;
        }
        if (a.push_world) __threadfence_system();  // this thread's peer stores, before the CTA counts itself in
    } else if (warp == kWarpRaw) {
        // ---------------- TMA producer of the raw weight tile ----------------
        if (lane == 0) {
            uint32_t g = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const int row0 = (int)(((tile / ksplit) % row_tiles) * kBM);
                const uint32_t kb0 = (tile % ksplit) * nkb;
                for (uint32_t kb = 0; kb < nkb; ++kb, ++g) {
                    const uint32_t s = ring<kRawStages>::stage(g);
                    if (ring<kRawStages>::must_wait_empty(g))
                        ok = mbar_wait(&raw_empty[s], ring<kRawStages>::empty_parity(g), abort_s);
                    if (!ok) break;
                    mbar_expect_tx(&raw_full[s], L::kRawBytes);
                    tma_load_2d(sRaw + s * L::kRawBytes, &wmap, (int)((kb0 + kb) * kBK), row0, &raw_full[s]);
                }
            }
            // Giving up with copies still in flight: let them land before the CTA's memory goes away.
            if (!ok)
                for (uint32_t i = 0; i < (uint32_t)kRawStages && i < g; ++i)
                    mbar_wait(&raw_full[ring<kRawStages>::stage(g - 1 - i)], ring<kRawStages>::full_parity(g - 1 - i),
                              abort_s);
        }
    } else if (warp == kWarpTok) {
        // ---------------- TMA producer of the token sub-tiles ----------------
        if (lane == 0) {
            uint32_t g = 0;
            bool ok = true;
            tmdev::pdl_wait();  // the f16 copy of X is the predecessor's output
            for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x) {
                const uint32_t tok0 = (tile / ksplit / row_tiles) * kTB;
                const uint32_t kb0 = (tile % ksplit) * nkb;
                // A sub-tile wholly past the batch is neither loaded nor multiplied.
                const uint32_t subs = tok0 + BN < a.batch ? (uint32_t)kIssuers : 1u;
                for (uint32_t kb = 0; kb < nkb; ++kb, ++g) {
                    const uint32_t s = ring<kStages>::stage(g);
                    if (ring<kStages>::must_wait_empty(g))
                        ok = mbar_wait(&empty[s], ring<kStages>::empty_parity(g), abort_s);
                    if (!ok) break;
                    mbar_expect_tx(&full[s], subs * L::kSubBytes);
                    for (uint32_t sub = 0; sub < subs; ++sub)
                        tma_load_2d(sB + s * L::kBBytes + sub * L::kSubBytes, &xmap, (int)((kb0 + kb) * kBK),
                                    (int)(tok0 + sub * BN), &full[s]);
                }
            }
            if (!ok)
                for (uint32_t i = 0; i < (uint32_t)kStages && i < g; ++i)
                    mbar_wait(&full[ring<kStages>::stage(g - 1 - i)], ring<kStages>::full_parity(g - 1 - i), abort_s);
        }
    } else {
        // ---------------- MMA issuers ----------------
        // Issuer `sub` multiplies the shared A stage by its own token sub-tile into its own accumulator.
        // Stage indices and parities advance by increment: no divisions, no descriptor built from scratch.
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(kBM, BN);
            const uint32_t sub = (uint32_t)(warp - kWarpMma);
            const uint64_t db0 = umma_desc(smem_u32(sB + sub * L::kSubBytes));
            const uint32_t db_lo = (uint32_t)db0, db_hi = (uint32_t)(db0 >> 32);
            const uint32_t ta0 = tmem_base + L::kACol0, d_tmem = tmem_base + sub * BN;
            uint32_t it = 0, st = 0, par = 0;
            bool ok = true;
            for (uint32_t tile = blockIdx.x; tile < n_tiles && ok; tile += gridDim.x, ++it) {
                const bool live = (tile / ksplit / row_tiles) * kTB + sub * BN < a.batch;  // else: the barrier protocol only
                if (it >= 1u) ok = mbar_wait(acc_empty, (it - 1u) & 1u, abort_s);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                uint32_t accumulate = 0u;
                for (uint32_t kb = 0; kb < nkb; ++kb) {
                    ok = mbar_wait(&full[st], par, abort_s);
                    if (!ok) break;
                    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                    if (live) umma_f16_ts_x4(d_tmem, ta0 + st * 32u, db_lo + st * (L::kBBytes >> 4), db_hi, idesc, accumulate);
                    accumulate = 1u;
                    umma_commit(&empty[st]);  // frees the stage once this issuer's MMAs have read it
                    if (++st == (uint32_t)kStages) {
                        st = 0;
                        par ^= 1u;
                    }
                }
                if (ok) umma_commit(&acc_full[sub]);  // fires when every MMA of the tile has completed
            }
        }
    }
    // ---------------- teardown: everyone meets, tensor memory goes back ----------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && *abort_s) atomicOr(a.abort_flag, 1u);
    if (a.push_world) {
        __shared__ uint32_t s_flag[2];
        tm_symm_finish(a.peer, a.push_tail, a.push_world, a.push_rank, s_flag);
    }
    if (warp == kWarpMma) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"(L::kTmemCols)
                     : "memory");
    }
}

// f32 -> f16 copy of the activations (round to nearest even), the TMA source.
__global__ void x_to_f16_kernel(const float *x, __half *out, size_t n) {
    tmdev::pdl_wait();  // x is the predecessor's output; the workspace may still be read by the GEMM before
    tmdev::pdl_trigger();
    for (size_t i = ((size_t)blockIdx.x * blockDim.x + threadIdx.x) * 4; i < n; i += (size_t)gridDim.x * blockDim.x * 4) {
        if (i + 3 < n && (((size_t)(x + i)) & 15u) == 0) {
            const float4 v = *(const float4 *)(x + i);
            *(__half2 *)(out + i) = __floats2half2_rn(v.x, v.y);
            *(__half2 *)(out + i + 2) = __floats2half2_rn(v.z, v.w);
        } else {
            for (size_t j = i; j < n && j < i + 4; ++j) out[j] = __float2half_rn(x[j]);
        }
    }
}

// The same copy with the producer's elementwise step folded in, one CTA per token row:
// RMS norm times a weight vector, or activation(x) * up (the gated-FFN product).
template <int PRO>
__global__ void __launch_bounds__(256) x_prep_f16_kernel(const float *x, const float *pro, __half *out, uint32_t cols,
                                                          float eps) {
    __shared__ float red[8];
    tmdev::pdl_wait();  // x is the predecessor's output; the workspace may still be read by the GEMM before
    tmdev::pdl_trigger();
    const float *xr = x + (size_t)blockIdx.x * cols;
    __half *orow = out + (size_t)blockIdx.x * cols;
    float inv = 1.0f;
    if (PRO == TM_CUDA_PRO_RMSNORM) {
        float ss = 0.0f;
        for (uint32_t c = threadIdx.x; c < cols; c += 256) ss = fmaf(xr[c], xr[c], ss);
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = ss;
        __syncthreads();
        float tot = 0.0f;
#pragma unroll
        for (int w = 0; w < 8; ++w) tot += red[w];
        inv = 1.0f / sqrtf(tot / (float)cols + eps);
    }
    const float *pr = PRO == TM_CUDA_PRO_RMSNORM ? pro : PRO == TM_CUDA_PRO_NONE ? xr : pro + (size_t)blockIdx.x * cols;
    auto one = [&](float v, float p) -> float {
        if (PRO == TM_CUDA_PRO_RMSNORM) return v * inv * p;
        if (PRO == TM_CUDA_PRO_SILU_MUL) return tmdev::silu_f(v) * p;
        if (PRO == TM_CUDA_PRO_GELU_MUL) return tmdev::gelu_tanh_f(v) * p;
        return v;
    };
    if ((cols & 3u) == 0u && ((((size_t)xr) | ((size_t)pr) | ((size_t)orow << 1)) & 15u) == 0u) {
        for (uint32_t c = threadIdx.x * 4u; c < cols; c += 1024u) {  // four columns per thread and trip
            const float4 v = *(const float4 *)(xr + c), p = *(const float4 *)(pr + c);
            const __half2 lo = __floats2half2_rn(one(v.x, p.x), one(v.y, p.y));
            const __half2 hi = __floats2half2_rn(one(v.z, p.z), one(v.w, p.w));
            *(uint2 *)(orow + c) = make_uint2(*(const uint32_t *)&lo, *(const uint32_t *)&hi);
        }
    } else {
        for (uint32_t c = threadIdx.x; c < cols; c += 256) orow[c] = __float2half_rn(one(xr[c], pr[c]));
    }
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

encode_tiled_fn get_encode_tiled() {
    static encode_tiled_fn fn = nullptr;
    static bool tried = false;
    if (!tried) {
        tried = true;
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            fn = (encode_tiled_fn)p;
        else
            cudaGetLastError();
    }
    return fn;
}

template <int BN>
cudaError_t launch_mma(tm_cuda_ctx *ctx, const CUtensorMap &wmap, const CUtensorMap &xmap, const mma_args &a, int grid) {
    const int device = ctx->device;
    static std::atomic<bool> attr_done[64] = {};  // per device; contexts of a process share it
    if (device < 0 || device >= 64 || !attr_done[device].load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(q8_gemm_mma_kernel<BN>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                                   (int)mma_smem<BN>::kBytes);
        if (e != cudaSuccess) return e;
        if (device >= 0 && device < 64) attr_done[device].store(true, std::memory_order_release);
    }
    return tm_launch_pdl(ctx, q8_gemm_mma_kernel<BN>, dim3(grid), dim3(kMmaThreads), mma_smem<BN>::kBytes, wmap, xmap, a);
}

}  // namespace

extern "C" {

int tm_cuda_mma_workspace_reserve(tm_cuda_ctx *ctx, size_t bytes, char *err, size_t err_cap) {
    TM_ENTER();
    if (bytes <= ctx->mma_scratch_bytes) return TM_CUDA_OK;
    if (ctx->group_open)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "the tensor-core GEMM workspace (%zu bytes) must be reserved before a dispatch group opens",
                       bytes);
    TM_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    if (ctx->mma_scratch) {
        cudaFree(ctx->mma_scratch);
        ctx->allocated.fetch_sub(ctx->mma_scratch_bytes);
        ctx->mma_scratch = nullptr;
        ctx->mma_scratch_bytes = 0;
    }
    void *p = nullptr;
    const size_t total = tm_round_up(bytes, 256) + 256;  // + the abort flag word
    if (cudaMalloc(&p, total) != cudaSuccess) {
        cudaGetLastError();
        return tm_fail(err, err_cap, TM_CUDA_ERR_ALLOC, "allocating the %zu-byte GEMM workspace failed", total);
    }
    TM_CUDA_TRY(cudaMemsetAsync(p, 0, total, ctx->stream));
    ctx->mma_scratch = (unsigned char *)p;
    ctx->mma_scratch_bytes = bytes;
    ctx->allocated.fetch_add(bytes);
    return TM_CUDA_OK;
}

// The f16 copy of X, then the split-K slots and counters.
size_t tm_cuda_mma_workspace_bytes(uint32_t cols, uint32_t batch) {
    return tm_round_up((size_t)cols * batch * 2, 256) + kSplitBytes;
}

// Grows the f16 workspace when the call needs more (outside a dispatch group only).
static int mma_ensure_workspace(tm_cuda_ctx *ctx, uint32_t cols, uint32_t batch, char *err, size_t err_cap) {
    const size_t need = tm_cuda_mma_workspace_bytes(cols, batch);
    bool small;
    {
        if (!ctx) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "null context");
        std::lock_guard<std::mutex> lock(ctx->mu);
        small = ctx->mma_scratch_bytes < need;
    }
    return small ? tm_cuda_mma_workspace_reserve(ctx, need, err, err_cap) : TM_CUDA_OK;
}

// The GEMM launch proper: the f16 copy of X is already in the workspace.  Called with the context locked.
struct mma_push {
    float *const *peer = nullptr;
    uint32_t world = 0, rank = 0, off = 0, tail = 0;
};

static int mma_launch(tm_cuda_ctx *ctx, const tm_cuda_buffer *w, uint32_t rows, uint32_t cols, uint32_t batch,
                      float *const y[3], const uint32_t part_end[3], int accumulate, char *err, size_t err_cap,
                      const mma_push &push = mma_push()) {
    encode_tiled_fn encode = get_encode_tiled();
    if (!encode)
        return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "the driver does not export cuTensorMapEncodeTiled");
    __half *xh = (__half *)ctx->mma_scratch;
    uint32_t *abort_flag = (uint32_t *)(ctx->mma_scratch + tm_round_up(ctx->mma_scratch_bytes, 256));
    // Sub-tile width BN (a tile is 128 rows x 2*BN tokens): the one whose rounds of the persistent
    // grid cost the fewest cycles.  Fitted to measurements: a K step takes the larger of the
    // tensor-pipe time plus hand-over (4*BN + 94 cycles for the two issuers' eight MMAs) and the
    // issuing threads' own 669 cycles; the unhidden epilogue adds about 30 cycles per token column.
    const uint32_t row_tiles = (rows + kBM - 1) / kBM, sms = (uint32_t)ctx->sm_count;
    int bn = 64;
    {
        const uint64_t nkb = (cols + kBK - 1) / kBK;
        uint64_t best = ~0ull;
        for (int cand : {192, 128, 64}) {
            const uint32_t tiles = row_tiles * ((batch + 2 * cand - 1) / (2 * cand));
            const uint64_t step = 4 * cand + 94 > 669 ? 4 * cand + 94 : 669;
            const uint64_t cost = (uint64_t)((tiles + sms - 1) / sms) * (nkb * step + 30ull * 2 * cand);
            if (cost < best) {
                best = cost;
                bn = cand;
            }
        }
    }
    CUtensorMap xmap, wmap;
    const cuuint32_t estr[2] = {1, 1};
    {
        const cuuint64_t gdim[2] = {cols, batch};
        const cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
        const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)bn};
        const CUresult cr = encode(&xmap, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)xh, gdim, gstride, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS)
            return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "cuTensorMapEncodeTiled (tokens) failed (%d)", (int)cr);
    }
    {
        // The int8 plane as bytes, 64 x 128 boxes, 64-byte swizzle; rows and columns past the end read as zero.
        const cuuint64_t gdim[2] = {cols, rows};
        const cuuint64_t gstride[1] = {(cuuint64_t)cols};
        const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)kBM};
        const CUresult cr = encode(&wmap, CU_TENSOR_MAP_DATA_TYPE_UINT8, 2, (void *)w->qp, gdim, gstride, box, estr,
                                   CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_64B,
                                   CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (cr != CUDA_SUCCESS)
            return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "cuTensorMapEncodeTiled (weights) failed (%d)", (int)cr);
    }
    mma_args a;
    a.d = (const __half *)w->dp;
    for (int p = 0; p < 3; ++p) {
        a.y[p] = y[p];
        a.part_end[p] = part_end[p];
    }
    a.accumulate = accumulate ? 1u : 0u;
    // Split K: the K range of every output tile is cut into `ksplit` equal parts when that shortens the
    // longest CTA's run -- rounds of the persistent grid x (K steps of a part + the fixed cost of a tile,
    // about 4 steps, + 2 for the ordered reduction) -- and the parts' accumulators fit the workspace
    // (never for the pushing form).
    a.ksplit = 1;
    const uint32_t tile_tokens = batch < 2u * (uint32_t)bn ? (batch + 31u) / 32u * 32u : 2u * (uint32_t)bn;
    a.kslot = 128u * tile_tokens;
    {
        const uint32_t out_tiles = row_tiles * ((batch + 2 * bn - 1) / (2 * bn)), nkb = (cols + kBK - 1) / kBK;
        static const bool off = [] { const char *e = getenv("TM_CUDA_MMA_SPLITK"); return e && e[0] == '0'; }();
        if (!off && push.world == 0 && bn <= 128 && cols % kBK == 0 && out_tiles * 16 <= kSplitCountBytes &&
            ctx->mma_scratch_bytes >= kSplitBytes) {
            const uint64_t whole = (uint64_t)((out_tiles + sms - 1) / sms) * (nkb + 4);
            uint64_t best = whole;
            for (uint32_t cand : {2u, 3u, 4u, 6u, 8u}) {
                if (nkb % cand != 0 || nkb / cand < 4) continue;
                if ((uint64_t)out_tiles * cand * a.kslot > (uint64_t)kSplitSlots * kSplitSlotFloats) continue;
                const uint64_t cost = (uint64_t)((out_tiles * cand + sms - 1) / sms) * (nkb / cand + 6);
                if (cost < best && cost * 10 < whole * 9) {  // a split has to pay for its reduction
                    best = cost;
                    a.ksplit = cand;
                }
            }
        }
    }
    unsigned char *split_base = ctx->mma_scratch + ((ctx->mma_scratch_bytes >= kSplitBytes ? ctx->mma_scratch_bytes - kSplitBytes : 0) & ~(size_t)255);
    a.kpart = (float *)split_base;
    a.kcount = (uint32_t *)(split_base + (size_t)kSplitSlots * kSplitSlotFloats * 4);
    a.peer = push.peer;
    a.push_world = push.world;
    a.push_rank = push.rank;
    a.push_off = push.off;
    a.push_tail = push.tail;
    a.rows = rows;
    a.cols = cols;
    a.batch = batch;
    a.abort_flag = abort_flag;
    ctx->mma_last_bn = bn;
    ctx->mma_last_ksplit = (int)a.ksplit;
    const uint32_t n_tiles = row_tiles * ((batch + 2 * bn - 1) / (2 * bn)) * a.ksplit;
    const int grid = (int)(n_tiles < (uint32_t)ctx->sm_count ? n_tiles : (uint32_t)ctx->sm_count);
    TM_CUDA_TRY(bn == 192   ? launch_mma<192>(ctx, wmap, xmap, a, grid)
                : bn == 128 ? launch_mma<128>(ctx, wmap, xmap, a, grid)
                            : launch_mma<64>(ctx, wmap, xmap, a, grid));
    return TM_CUDA_OK;
}

int tm_cuda_q8_0_gemm_mma(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t rows,
                          uint32_t cols, uint32_t batch, uint32_t x_off, uint32_t y_off, char *err, size_t err_cap) {
    if (batch >= 1 && (batch < 3 || (batch < 9 && cols < 2048))) {
        // One or two tokens (up to eight on a narrow matrix) are served by the exact integer-tensor-core
        // GEMV, which is tighter and as fast there; its per-token work on every weight chunk makes it
        // issue-bound beyond that (4096 x 12288 at 8 tokens: 196 us against 28 us here).
        return tm_cuda_q8_0_gemm(ctx, w, x, y, rows, cols, batch, x_off, y_off, err, err_cap);
    }
    {
        const int rc = mma_ensure_workspace(ctx, cols, batch, err, err_cap);
        if (rc != TM_CUDA_OK) return rc;
    }
    TM_ENTER();
    int rc = tm_check_packed(ctx, w, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    if (batch == 0 || batch > TM_CUDA_GEMM_MMA_MAX_BATCH)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "batch %u outside 1..%u", batch, TM_CUDA_GEMM_MMA_MAX_BATCH);
    TM_CHECK_BUF(x, ((size_t)x_off + (size_t)batch * cols) * 4, "activation");
    TM_CHECK_BUF(y, ((size_t)y_off + (size_t)batch * rows) * 4, "output");
    TM_OP_BEGIN("q8_0_gemm_mma");
    const size_t n = (size_t)batch * cols;
    const int cgrid = (int)((n / 4 + 255) / 256 > 148 * 8 ? 148 * 8 : (n / 4 + 255) / 256);
    TM_CUDA_TRY(tm_launch_pdl(ctx, x_to_f16_kernel, dim3(cgrid < 1 ? 1 : cgrid), dim3(256), 0,
                              (const float *)x->dev + x_off, (__half *)ctx->mma_scratch, n));
    float *const ys[3] = {(float *)y->dev + y_off, nullptr, nullptr};
    const uint32_t ends[3] = {rows, rows, rows};
    rc = mma_launch(ctx, w, rows, cols, batch, ys, ends, 0, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    TM_OP_END(2);
}

int tm_cuda_q8_0_gemm_mma_fused(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, uint32_t rows, uint32_t cols,
                                uint32_t batch, uint32_t n_parts, tm_cuda_buffer *const *y_parts,
                                const uint32_t *part_rows, int prologue, tm_cuda_buffer *pro, float eps, int epilogue,
                                char *err, size_t err_cap) {
    {
        const int rc = mma_ensure_workspace(ctx, cols, batch, err, err_cap);
        if (rc != TM_CUDA_OK) return rc;
    }
    TM_ENTER();
    int rc = tm_check_packed(ctx, w, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    if (batch == 0 || batch > TM_CUDA_GEMM_MMA_MAX_BATCH)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "batch %u outside 1..%u", batch, TM_CUDA_GEMM_MMA_MAX_BATCH);
    if (n_parts < 1 || n_parts > 3 || !y_parts || !part_rows)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "1 to 3 output parts, got %u", n_parts);
    if (prologue < TM_CUDA_PRO_NONE || prologue > TM_CUDA_PRO_GELU_MUL ||
        (epilogue != TM_CUDA_EPI_STORE && epilogue != TM_CUDA_EPI_ADD))
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "unknown prologue %d / epilogue %d", prologue, epilogue);
    float *ys[3] = {nullptr, nullptr, nullptr};
    uint32_t ends[3] = {rows, rows, rows}, sum = 0;
    for (uint32_t p = 0; p < n_parts; ++p) {
        if (part_rows[p] == 0 || (p + 1 < n_parts && part_rows[p] % kBM != 0))
            return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                           "part %u has %u rows: every part but the last must be a multiple of %d", p, part_rows[p], kBM);
        TM_CHECK_BUF(y_parts[p], (size_t)batch * part_rows[p] * 4, "output part");
        ys[p] = (float *)y_parts[p]->dev;
        sum += part_rows[p];
        ends[p] = sum;
    }
    if (sum != rows) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "parts cover %u of %u rows", sum, rows);
    TM_CHECK_BUF(x, (size_t)batch * cols * 4, "activation");
    if (prologue == TM_CUDA_PRO_RMSNORM) TM_CHECK_BUF(pro, (size_t)cols * 4, "norm weight");
    else if (prologue != TM_CUDA_PRO_NONE) TM_CHECK_BUF(pro, (size_t)batch * cols * 4, "gate operand");
    TM_OP_BEGIN("q8_0_gemm_mma_fused");
    __half *xh = (__half *)ctx->mma_scratch;
    const float *xp = (const float *)x->dev, *pp = pro ? (const float *)pro->dev : nullptr;
    switch (prologue) {
        case TM_CUDA_PRO_RMSNORM:
            TM_CUDA_TRY(tm_launch_pdl(ctx, x_prep_f16_kernel<TM_CUDA_PRO_RMSNORM>, dim3(batch), dim3(256), 0, xp, pp, xh, cols, eps));
            break;
        case TM_CUDA_PRO_SILU_MUL:
            TM_CUDA_TRY(tm_launch_pdl(ctx, x_prep_f16_kernel<TM_CUDA_PRO_SILU_MUL>, dim3(batch), dim3(256), 0, xp, pp, xh, cols, eps));
            break;
        case TM_CUDA_PRO_GELU_MUL:
            TM_CUDA_TRY(tm_launch_pdl(ctx, x_prep_f16_kernel<TM_CUDA_PRO_GELU_MUL>, dim3(batch), dim3(256), 0, xp, pp, xh, cols, eps));
            break;
        default:
            TM_CUDA_TRY(tm_launch_pdl(ctx, x_prep_f16_kernel<TM_CUDA_PRO_NONE>, dim3(batch), dim3(256), 0, xp, pp, xh, cols, eps));
    }
    rc = mma_launch(ctx, w, rows, cols, batch, ys, ends, epilogue == TM_CUDA_EPI_ADD, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    TM_OP_END(2);
}

int tm_cuda_q8_0_gemm_mma_push(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *dst,
                               uint32_t rows, uint32_t cols, uint32_t batch, char *err, size_t err_cap) {
    {
        const int rc = mma_ensure_workspace(ctx, cols, batch, err, err_cap);
        if (rc != TM_CUDA_OK) return rc;
    }
    TM_ENTER();
    int rc = tm_check_packed(ctx, w, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    if (batch == 0 || batch > TM_CUDA_GEMM_MMA_MAX_BATCH)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "batch %u outside 1..%u", batch, TM_CUDA_GEMM_MMA_MAX_BATCH);
    tm_cuda_buffer *root = dst && dst->parent ? dst->parent : dst;
    if (!dst || ctx->live.find(dst) == ctx->live.end() || !root || !root->symm)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "the target is not (a view of) a symmetric buffer of this context");
    const tm_symm_state *st = (const tm_symm_state *)root->symm;
    TM_CHECK_BUF(x, (size_t)batch * cols * 4, "activation");
    TM_CHECK_BUF(dst, (size_t)batch * rows * (size_t)st->world * 4, "gathered output");
    const size_t dst_off = (size_t)(dst->dev - root->dev);
    if (dst_off % 16 != 0) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "target view is not 16-byte aligned");
    TM_OP_BEGIN("q8_0_gemm_mma_push");
    const size_t n = (size_t)batch * cols;
    const int cgrid = (int)((n / 4 + 255) / 256 > 148 * 8 ? 148 * 8 : (n / 4 + 255) / 256);
    TM_CUDA_TRY(tm_launch_pdl(ctx, x_to_f16_kernel, dim3(cgrid < 1 ? 1 : cgrid), dim3(256), 0, (const float *)x->dev,
                              (__half *)ctx->mma_scratch, n));
    float *const ys[3] = {(float *)dst->dev, nullptr, nullptr};  // unused by the pushing epilogue
    const uint32_t ends[3] = {rows, rows, rows};
    mma_push push;
    push.peer = (float *const *)st->d_peer;
    push.world = (uint32_t)st->world;
    push.rank = (uint32_t)st->rank;
    push.off = (uint32_t)(dst_off / 4);
    push.tail = (uint32_t)(st->payload / 4);
    rc = mma_launch(ctx, w, rows, cols, batch, ys, ends, 0, err, err_cap, push);
    if (rc != TM_CUDA_OK) return rc;
    TM_OP_END(2);
}

// Token sub-tile width (64, 128 or 192) of the kernel instantiation the last GEMM launch used.
int tm_cuda_mma_last_tile(tm_cuda_ctx *ctx) {
    if (!ctx) return 0;
    std::lock_guard<std::mutex> lock(ctx->mu);
    return ctx->mma_last_bn;
}

// K parts per output tile of the last GEMM launch (1: no split).
int tm_cuda_mma_last_split(tm_cuda_ctx *ctx) {
    if (!ctx) return 0;
    std::lock_guard<std::mutex> lock(ctx->mu);
    return ctx->mma_last_ksplit;
}

// 1 when a tensor-core GEMM on this context ever gave up a bounded wait.
int tm_cuda_mma_aborted(tm_cuda_ctx *ctx) {
    if (!ctx) return 0;
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (!ctx->mma_scratch) return 0;
    uint32_t v = 0;
    cudaSetDevice(ctx->device);
    cudaStreamSynchronize(ctx->stream);
    cudaMemcpy(&v, ctx->mma_scratch + tm_round_up(ctx->mma_scratch_bytes, 256), 4, cudaMemcpyDeviceToHost);
    return v != 0;
}

}  // extern "C"
