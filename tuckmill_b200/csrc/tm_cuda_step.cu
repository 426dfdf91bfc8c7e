// A whole decode step as ONE persistent kernel.
//
// The reference encodes a decode step as one command buffer of ~17 dispatches per
// layer (crates/tuckcore/src/qwen35_gpu.rs:66-86, engine/metal.rs:2381-2449); the
// graph form of this library replays ~5 kernels per layer.  At batch 1 a projection
// of a small decoder is 2-6 MB: a kernel per projection spends most of its time
// starting, staging its input and draining, and the weight stream stops at every
// kernel boundary.  Here the operators of a step are recorded into a PROGRAM
// (tm_cuda_begin_program ... tm_cuda_end_program) and one kernel, one CTA per SM,
// walks it:
//
//   * The weights of a step never depend on its activations, so a producer warp
//     per CTA streams them -- in program order, across operator boundaries -- into a
//     ring of shared-memory stages (one cp.async.bulk.tensor copy of 16 rows x 1024
//     bytes per stage -- sixteen row-sized bulk copies per stage kept the whole chip
//     at 1.6 TB/s -- plus cp.async for the f16 block scales, completion on an
//     mbarrier per stage).  While the
//     consumers wait for the activations of operator i, the weights of operators
//     i+1, i+2, ... are already landing: the HBM stream never stops.
//   * An operator's output rows are cut into units of 16 rows x all columns, dealt
//     round-robin over the CTAs (the deal continues across operators, so every CTA
//     streams the same number of bytes per step).  The 8 consumer warps of a CTA
//     split a unit's columns, multiply with the integer tensor-core form of the
//     GEMV kernel (tm_cuda_q8.cu: s8 x s8 -> s32 against signed digits of the f32
//     activations), add their partial row sums in a fixed order and store --
//     a row has exactly one owner, results are deterministic.
//   * There is NO grid barrier.  A vector that one operator produces and a later
//     one consumes travels as 8-byte words {f32 value, sequence number}, each
//     written with one 64-bit store: a consumer polls the words it needs until
//     they carry the number of (this launch, the producing operator), so the value
//     and its "ready" flag arrive together and a dependent operator starts one L2
//     round trip after the last row it needs was stored (a barrier measured 3.4 us
//     per operator on this part, the polled words about 0.5).  Every flagged
//     region is written once per launch, so nothing is overwritten while it is
//     still being read.  Every poll is bounded; when one runs out the CTA raises a
//     status bit, stops producing and returns, and the others follow.
//
// Attention is the latency-optimised decode kernel of tm_cuda_ops.cu (same
// arithmetic and key split) run by groups of four warps, two (KV head, key
// split) items per CTA at a time; the splits of a KV head are merged by the group
// that holds the newest key, which polls the other groups' flagged partials.
#include <cuda.h>

#include <cstdlib>

#include "tm_cuda_internal.cuh"
#include "tm_cuda_device.cuh"

namespace {

using tmdev::gelu_tanh_f;
using tmdev::silu_f;
typedef unsigned long long u64;

constexpr int kCWarps = 8;                      // consumer warps (288 threads leave each thread 168 registers: with
                                                // the shared-memory carve-out at its maximum L1 is ~28 KB, and a
                                                // spilled register costs an L2 round trip)
constexpr int kCThreads = kCWarps * 32;         // 256
constexpr int kStepThreads = kCThreads + 32;    // + the producer warp
constexpr uint32_t kChunkCols = 64;             // columns one pair of m16n8k32 MMAs covers
constexpr uint32_t kStageChunks = 16;           // chunks per ring stage: 16 rows x 1024 columns
constexpr uint32_t kStageCols = kStageChunks * kChunkCols;  // 1024
constexpr uint32_t kQuantBytes = 16 * kStageCols;  // 16 dense rows, written by ONE tensor-map copy
constexpr uint32_t kScaleStride = 80;           // 32 f16 scales of a row + 16: rows land in different banks
constexpr uint32_t kSlotBytes = kQuantBytes + 16 * kScaleStride;  // 17664, a multiple of 128
constexpr uint32_t kMaxSlots = 12;
constexpr uint32_t kMaxQuads = 12;              // activation quads per consumer thread: cols <= 12288
constexpr uint32_t kNormQuads = 8;              // ... of a vector that is RMS-normed on the way in: cols <= 8192
constexpr uint32_t kPollQuads = 4;              // quads a thread polls for at a time
constexpr uint32_t kUnitBatch = 8;              // units a CTA multiplies between two syncs of its consumer warps
constexpr uint32_t kAttnSub = 10752;            // shared memory of one attention warp group
constexpr uint32_t kAttnSplit = 64;             // keys per attention item (the fast decode kernel's split)
constexpr uint32_t kDescWords = 64;             // a descriptor is copied to shared memory as 64 x 4 bytes
constexpr uint32_t kTailBytes = 2 * kMaxSlots * 8 + 2 * kUnitBatch * kCWarps * 16 * 4 + 32 * 4 + 2 * kDescWords * 4 + 64;
constexpr uint32_t kArgmaxNone = 0xFFFFFFFFu;

enum : uint32_t { STEP_EMBED = 1, STEP_GEMV = 2, STEP_ATTN = 3, STEP_ARGMAX = 4, STEP_NORM_ADD = 5, STEP_POS_ADD = 6 };

// One recorded operator (256 bytes).  Pointer and integer slots by kind:
//   GEMV      p0 q plane, p1 scale plane, p2 x, p3 y, p4 prologue operand; rows, cols, prologue, epilogue, eps
//             flagged sources: in0 x, in1 prologue operand (activation forms), in2 the old y (accumulate)
//   EMBED     p0 q plane, p1 scale plane, p2 ids, p3 position (or null), p4 out; rows, cols, u0 slot, u1 bias,
//             u2 ids length, scale
//   ATTN      p0 q, p1 k, p2 v, p3 q norm, p4 k norm, p5 inv_freq, p6 k cache, p7 v cache, p8 out, p10 position,
//             p11 status; u0 heads, u1 kv heads, u2 head dim, u3 capacity, u4 window; eps, scale
//             flagged sources: in0 q, in1 k, in2 v
//   ARGMAX    p0 x, p1 out, p2 position (or null), p3 mirror (or null); u0 n, u1 base slot, u2 out capacity
//             flagged source: in0 x
//   NORM_ADD  p0 p, p1 weight, p2 x; cols, eps; flagged sources: in0 p, in1 the old x
//   POS_ADD   p0 counter; u0 delta
// `out` is the flagged copy of the operator's output vector; a null source means the plain buffer
// was complete before the launch (written by an earlier launch or by the host).
struct step_op {
    uint32_t kind, first_cta, rows, cols, prologue, epilogue;
    float eps, scale;
    const void *p[12];
    uint32_t u[6];
    u64 *out;               // flagged output words
    const u64 *in[3];       // flagged sources
    uint32_t in_op[3];      // the operator that produces each source (its index names the sequence number)
    uint32_t write_plain;   // also store the plain vector (no later operator of the program overwrites it)
    uint32_t row_stride;    // GEMV: bytes between the rows of a stage in shared memory, min(1024, cols)
    const void *wmap;       // GEMV: tensor map of the int8 plane as [rows][cols / 4] u32, box 16 rows x row_stride
    uint32_t pad[10];
};
static_assert(sizeof(step_op) == kDescWords * 4, "descriptor size");

struct step_params {
    const step_op *ops;
    uint32_t n_ops;
    uint32_t seq_base;      // sequence number of operator 0 in this launch (never 0; differs from the last launch's)
    uint32_t seq_skew;      // added to the number a consumer expects: non-zero only in the run-out test
    uint32_t *arrivals;     // CTAs that finished all operators before a position update, monotonic
    uint32_t arrivals_base;
    uint32_t *status;       // bit 0: a wait for activations ran out; bit 1: a weight-stage wait ran out
    u64 *argmax_ll;         // [2 * grid] flagged per-CTA candidates of the greedy choice
    u64 *attn_ll;           // flagged attention partials, shared by all attention operators
    uint32_t n_slots, xs_bytes, spin_limit;
    uint32_t l2_ahead;      // stages the L2 prefetch runs ahead of the ring
    u64 *trace;             // optional: [n_ops][8] nanosecond stamps of CTA 0 (tm_cuda_program_trace)
};

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
__device__ __forceinline__ bool mbar_try(uint32_t addr, uint32_t parity) {
    uint32_t done;
    asm volatile(
        "{\n .reg .pred p;\n mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n selp.b32 %0, 1, 0, p;\n}\n"
        : "=r"(done)
        : "r"(addr), "r"(parity)
        : "memory");
    return done != 0;
}
// Bounded wait on a phase parity.  False when it gave up or the CTA is stopping; the caller skips
// the data.
__device__ __forceinline__ bool mbar_wait(uint64_t *bar, uint32_t parity, volatile uint32_t *flags, uint32_t limit,
                                          uint32_t *status) {
    const uint32_t addr = smem_u32(bar);
    for (uint32_t spin = 0; spin < limit; ++spin) {
        if (mbar_try(addr, parity)) return true;
        if ((spin & 255u) == 255u && flags[0]) return false;
    }
    flags[0] = 1u;
    atomicOr(status, 2u);
    return false;
}
__device__ __forceinline__ void trace_stamp(const step_params &P, uint32_t oi, int k) {
    if (P.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0) {
        u64 t;
        asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
        P.trace[(size_t)oi * 8 + k] = t;
    }
}
__device__ __forceinline__ void consumer_sync() { asm volatile("bar.sync 1, %0;" ::"n"(kCThreads) : "memory"); }
__device__ __forceinline__ void group_sync(int id) { asm volatile("bar.sync %0, 128;" ::"r"(id) : "memory"); }

// ---- flagged words ------------------------------------------------------------------------
// {f32 value | sequence number << 32}, stored and loaded as ONE 64-bit access, past L1.
__device__ __forceinline__ void ll_store(u64 *p, float v, uint32_t seq) {
    const u64 w = ((u64)seq << 32) | (u64)__float_as_uint(v);
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ void ll_store_u32(u64 *p, uint32_t v, uint32_t seq) {
    const u64 w = ((u64)seq << 32) | (u64)v;
    asm volatile("st.relaxed.gpu.global.u64 [%0], %1;" ::"l"(p), "l"(w) : "memory");
}
__device__ __forceinline__ u64 ll_load(const u64 *p) {
    u64 w;
    asm volatile("ld.relaxed.gpu.global.u64 %0, [%1];" : "=l"(w) : "l"(p) : "memory");
    return w;
}
struct ll_quad {
    u64 w[4];
};
__device__ __forceinline__ void ll_load_quad(const u64 *p, ll_quad &q) {  // 32-byte aligned
    asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(q.w[0]), "=l"(q.w[1]) : "l"(p) : "memory");
    asm volatile("ld.volatile.global.v2.u64 {%0,%1}, [%2];" : "=l"(q.w[2]), "=l"(q.w[3]) : "l"(p + 2) : "memory");
}
__device__ __forceinline__ bool ll_quad_ready(const ll_quad &q, uint32_t seq) {
    return (uint32_t)(q.w[0] >> 32) == seq && (uint32_t)(q.w[1] >> 32) == seq && (uint32_t)(q.w[2] >> 32) == seq &&
           (uint32_t)(q.w[3] >> 32) == seq;
}
__device__ __forceinline__ float4 ll_quad_values(const ll_quad &q) {
    return make_float4(__uint_as_float((uint32_t)q.w[0]), __uint_as_float((uint32_t)q.w[1]),
                       __uint_as_float((uint32_t)q.w[2]), __uint_as_float((uint32_t)q.w[3]));
}
// What every wait for activations does when it is not satisfied yet: count the poll, give up at the
// limit (status bit 0) or when the CTA or the program is already stopping.  True = keep polling.
__device__ __forceinline__ bool poll_again(const step_params &P, volatile uint32_t *flags, uint32_t &spin) {
    if (flags[0]) return false;
    if (++spin >= P.spin_limit) {
        flags[0] = 1u;
        atomicOr(P.status, 1u);
        return false;
    }
    if ((spin & 63u) == 63u) {
        uint32_t st;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(st) : "l"(P.status) : "memory");
        if (st) {
            flags[0] = 1u;
            return false;
        }
    }
    return true;
}
// One flagged value (bounded).
__device__ __forceinline__ float ll_wait(const step_params &P, const u64 *p, uint32_t seq, volatile uint32_t *flags) {
    uint32_t spin = 0;
    for (;;) {
        const u64 w = ll_load(p);
        if ((uint32_t)(w >> 32) == seq) return __uint_as_float((uint32_t)w);
        if (!poll_again(P, flags, spin)) return 0.0f;
    }
}

// D += A(16x32 s8, row) * B(32x8 s8, col), s32 accumulate.
__device__ __forceinline__ void mma_s8(int (&d)[4], int a0, int a1, int a2, int a3, int b0, int b1) {
    asm(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

__host__ __device__ inline uint32_t digit_plane(uint32_t cols) {
    const uint32_t pad = (cols + kChunkCols - 1u) / kChunkCols * kChunkCols;
    return pad % 128u == 0 ? pad + 64u : pad;
}
__host__ __device__ inline uint32_t stage_bytes_for(uint32_t cols) { return 3u * digit_plane(cols) + (cols / 32u) * 16u; }

// ---- activation staging -------------------------------------------------------------
// x (after the operator's elementwise prologue) as three planes of signed 8-bit digits against a
// power-of-two scale per 32-column block, plus the coefficients 2^(E - 21 + 8k) per block -- the B
// operand of the integer MMA (the digit-split GEMV is described at q8_gemv_kernel in tm_cuda_q8.cu).
// Sources produced inside this launch are polled as flagged words, four quads per thread at a time.

// Four consecutive activations (columns c..c+3, final values) -> digits and block coefficients.
// Eight adjacent lanes hold one 32-column block; whole warps call this together.
// Per block: E = exponent of the largest magnitude, T = round(v * 2^(21 - E)) (|T| <= 2^22), and T in
// balanced base 256: T + 0x808080 has the bytes a_k + 128, so one add and one xor give the three
// signed digits of an element as the bytes of a word; v = sum_k a_k 2^(E - 21 + 8k) to 2^-22 of the
// block's largest value.  (The stand-alone GEMV kernel splits into four 7-bit digits; here staging is
// repeated by every CTA for every operator, and this split costs a third of the instructions.)
__device__ __forceinline__ void digitize_quad(const float (&v)[4], uint32_t c, uint32_t cols, uint32_t plane,
                                              signed char *dig, float *coef, int lane) {
    float amax = 0.0f;
#pragma unroll
    for (int j = 0; j < 4; ++j)  // a non-finite value poisons its block (amax = inf -> NaN coefficient)
        amax = fmaxf(amax, fabsf(v[j]) <= 3.402823466e38f ? fabsf(v[j]) : INFINITY);
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
    amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
    if (c >= cols) return;
    const bool bad = !(amax <= 3.402823466e38f);
    int e = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127;
    e = e < -100 ? -100 : e > 100 ? 100 : e;  // blocks below 2^-100 digitise to (near) zero
    const float up = __uint_as_float((uint32_t)(127 + 21 - e) << 23);  // 2^(21 - E)
    uint32_t X[4];
#pragma unroll
    for (int j = 0; j < 4; ++j) X[j] = ((uint32_t)__float2int_rn(v[j] * up) + 0x808080u) ^ 0x808080u;
    *(uint32_t *)(dig + c) = __byte_perm(__byte_perm(X[0], X[1], 0x0040), __byte_perm(X[2], X[3], 0x0040), 0x5410);
    *(uint32_t *)(dig + plane + c) = __byte_perm(__byte_perm(X[0], X[1], 0x0051), __byte_perm(X[2], X[3], 0x0051), 0x5410);
    *(uint32_t *)(dig + 2u * plane + c) = __byte_perm(__byte_perm(X[0], X[1], 0x0062), __byte_perm(X[2], X[3], 0x0062), 0x5410);
    const int k = lane & 7;
    if (k < 4) {
        float sc = k < 3 ? __uint_as_float((uint32_t)(127 + e - 21 + 8 * k) << 23) : 0.0f;  // 2^(E - 21 + 8k)
        if (amax == 0.0f) sc = 0.0f;
        if (bad && k < 3) sc = __uint_as_float(0x7fc00000u);
        coef[(c >> 5) * 4u + k] = sc;
    }
}

// Polls (or plainly loads) this thread's quads i0 .. i0 + kPollQuads - 1 of one vector.
template <uint32_t NQ>
__device__ __forceinline__ void fetch_quads(const step_params &P, const float *plain, const u64 *ll, uint32_t seq,
                                            uint32_t i0, uint32_t cols, float fill, float4 (&out)[NQ],
                                            volatile uint32_t *flags) {
    constexpr uint32_t kPollQuads = NQ;
    const int tid = threadIdx.x;
    ll_quad q[kPollQuads];
    bool need[kPollQuads];
#pragma unroll
    for (uint32_t j = 0; j < kPollQuads; ++j) {
        const uint32_t c = ((i0 + j) * kCThreads + tid) * 4u;
        out[j] = make_float4(fill, fill, fill, fill);
        need[j] = false;
        if (c < cols) {
            if (ll) { need[j] = true; ll_load_quad(ll + c, q[j]); }
            else out[j] = __ldcg((const float4 *)(plain + c));
        }
    }
    if (!ll) return;
    uint32_t spin = 0;
    for (;;) {
        bool again = false;
#pragma unroll
        for (uint32_t j = 0; j < kPollQuads; ++j) {
            if (!need[j]) continue;
            if (ll_quad_ready(q[j], seq)) { out[j] = ll_quad_values(q[j]); need[j] = false; }
            else { ll_load_quad(ll + ((i0 + j) * kCThreads + tid) * 4u, q[j]); again = true; }
        }
        if (!again || !poll_again(P, flags, spin)) break;
    }
}

__device__ __forceinline__ void stage_activations(const step_params &P, const step_op &op, uint32_t oi, unsigned char *xs, float *red,
                                  volatile uint32_t *flags) {
    const uint32_t cols = op.cols, plane = digit_plane(cols);
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5;
    const float *x = (const float *)op.p[2], *pro = (const float *)op.p[4];
    const uint32_t xseq = P.seq_base + op.in_op[0] + P.seq_skew, pseq = P.seq_base + op.in_op[1] + P.seq_skew;
    const uint32_t prologue = op.prologue;
    signed char *dig = (signed char *)xs;
    float *coef = (float *)(xs + 3u * (size_t)plane);
    const uint32_t warp_col0 = (tid & ~31u) * 4u;  // first column of this warp's quad 0
    if (prologue == TM_CUDA_PRO_RMSNORM) {
        // The whole row waits for its sum of squares.  A thread keeps its first kKeepQuads quads in
        // registers (rows up to 2048 columns entirely); further quads are polled for the sum and
        // fetched again for the digits (valid by then: one more L2 trip, no more registers).
        constexpr uint32_t kKeepQuads = 2;
        float4 kept[kKeepQuads], wts[kKeepQuads];
#pragma unroll
        for (uint32_t i = 0; i < kKeepQuads; ++i) {
            const uint32_t c = (i * kCThreads + tid) * 4u;
            wts[i] = c < cols ? __ldg((const float4 *)(pro + c)) : make_float4(1.f, 1.f, 1.f, 1.f);
        }
        float sq = 0.0f;
        fetch_quads<kKeepQuads>(P, x, op.in[0], xseq, 0, cols, 0.0f, kept, flags);
#pragma unroll
        for (uint32_t j = 0; j < kKeepQuads; ++j) sq = tmdev::sumsq_quad(sq, kept[j]);
#pragma unroll 1
        for (uint32_t i0 = kKeepQuads; i0 < kNormQuads; i0 += kKeepQuads) {
            if (i0 * kCThreads * 4u + warp_col0 >= cols) break;
            float4 vs[kKeepQuads];
            fetch_quads<kKeepQuads>(P, x, op.in[0], xseq, i0, cols, 0.0f, vs, flags);
#pragma unroll
            for (uint32_t j = 0; j < kKeepQuads; ++j) sq = tmdev::sumsq_quad(sq, vs[j]);
        }
        trace_stamp(P, oi, 3);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
        if (lane == 0) red[warp] = sq;
        consumer_sync();
        float t = 0.0f;
#pragma unroll
        for (int w = 0; w < kCWarps; ++w) t += red[w];
        const float inv_rms = 1.0f / sqrtf(t / (float)cols + op.eps);
#pragma unroll
        for (uint32_t i = 0; i < kKeepQuads; ++i) {
            const uint32_t c = (i * kCThreads + tid) * 4u;
            if (i * kCThreads * 4u + warp_col0 < cols) {  // whole warps digitise together
                const float v[4] = {kept[i].x * inv_rms * wts[i].x, kept[i].y * inv_rms * wts[i].y,
                                    kept[i].z * inv_rms * wts[i].z, kept[i].w * inv_rms * wts[i].w};
                digitize_quad(v, c, cols, plane, dig, coef, lane);
            }
        }
#pragma unroll 1
        for (uint32_t i0 = kKeepQuads; i0 < kNormQuads; i0 += kKeepQuads) {
            if (i0 * kCThreads * 4u + warp_col0 >= cols) break;
            float4 vs[kKeepQuads];
            fetch_quads<kKeepQuads>(P, x, op.in[0], xseq, i0, cols, 0.0f, vs, flags);
#pragma unroll
            for (uint32_t j = 0; j < kKeepQuads; ++j) {
                const uint32_t c = ((i0 + j) * kCThreads + tid) * 4u;
                if ((i0 + j) * kCThreads * 4u + warp_col0 < cols) {
                    float4 w4 = make_float4(1.f, 1.f, 1.f, 1.f);
                    if (c < cols) w4 = __ldg((const float4 *)(pro + c));
                    const float v[4] = {vs[j].x * inv_rms * w4.x, vs[j].y * inv_rms * w4.y, vs[j].z * inv_rms * w4.z,
                                        vs[j].w * inv_rms * w4.w};
                    digitize_quad(v, c, cols, plane, dig, coef, lane);
                }
            }
        }
    } else {
        const bool act = prologue == TM_CUDA_PRO_SILU_MUL || prologue == TM_CUDA_PRO_GELU_MUL;
#pragma unroll 1
        for (uint32_t i0 = 0; i0 < kMaxQuads; i0 += kPollQuads) {
            if (i0 * kCThreads * 4u + warp_col0 >= cols) break;  // this warp has no more columns
            float4 vs[kPollQuads], ps[kPollQuads];
            fetch_quads<kPollQuads>(P, x, op.in[0], xseq, i0, cols, 0.0f, vs, flags);
            if (act) fetch_quads<kPollQuads>(P, pro, op.in[1], pseq, i0, cols, 1.0f, ps, flags);
            if (i0 == 0) trace_stamp(P, oi, 3);
#pragma unroll
            for (uint32_t j = 0; j < kPollQuads; ++j) {
                const uint32_t c = ((i0 + j) * kCThreads + tid) * 4u;
                if ((i0 + j) * kCThreads * 4u + warp_col0 < cols) {
                    float v[4] = {vs[j].x, vs[j].y, vs[j].z, vs[j].w};
                    if (act) {
                        const float pw[4] = {ps[j].x, ps[j].y, ps[j].z, ps[j].w};
#pragma unroll
                        for (int e = 0; e < 4; ++e)
                            v[e] = (prologue == TM_CUDA_PRO_SILU_MUL ? silu_f(v[e]) : gelu_tanh_f(v[e])) * pw[e];
                    }
                    digitize_quad(v, c, cols, plane, dig, coef, lane);
                }
            }
        }
    }
    consumer_sync();
}

// ---- one GEMV operator, consumer side ------------------------------------------------
// `n` counts the stages this CTA has consumed since the kernel began (the producer counts the same
// sequence): stage n sits in ring slot n % n_slots with phase parity (n / n_slots) & 1.
__device__ __forceinline__ void gemv_consume(const step_params &P, const step_op &op, uint32_t oi, unsigned char *xs,
                             unsigned char *slots, uint64_t *full, uint64_t *empty, float *partial,
                             volatile uint32_t *flags, uint32_t &n, uint32_t &pbuf) {
    const int tid = threadIdx.x, lane = tid & 31, warp = tid >> 5, g = lane >> 2, t4 = lane & 3;
    const uint32_t rows = op.rows, cols = op.cols, plane = digit_plane(cols);
    const uint32_t n_units = (rows + 15u) / 16u, n_chunks = cols / kChunkCols;
    const uint32_t n_stages = (n_chunks + kStageChunks - 1u) / kStageChunks;
    const bool b_live = (t4 >> 1) == (g >> 2) && (g & 3) < 3;  // B column g = (block g / 4, digit g % 4); three digits
    const uint32_t rs = op.row_stride;
    float *y = (float *)op.p[3];
    u64 *yl = op.out;
    const u64 *oldl = op.in[2];
    const bool add = op.epilogue == TM_CUDA_EPI_ADD, plain = op.write_plain != 0;
    const uint32_t seq = P.seq_base + oi, old_seq = P.seq_base + op.in_op[2] + P.seq_skew;
    const unsigned char *coef_base = xs + 3u * (size_t)plane;
    bool first_unit = true;
    const uint32_t u_first = (blockIdx.x + gridDim.x - op.first_cta) % gridDim.x;
    // Units in batches of up to kUnitBatch: every warp leaves its partial row sums of each unit in shared
    // memory, ONE sync ends the batch, then thread (unit j, row r) adds the warps' partials in order,
    // adds the residual value if the operator accumulates, and publishes the row.
    for (uint32_t u0 = u_first; u0 < n_units; u0 += gridDim.x * kUnitBatch) {
        const uint32_t left = (n_units - u0 + gridDim.x - 1u) / gridDim.x;
        const uint32_t nbu = left < kUnitBatch ? left : kUnitBatch;
        // the residual value of this thread's row, if any, travels while the batch is multiplied
        float old = 0.0f;
        u64 oldw = 0;
        const uint32_t my_row = (u0 + ((uint32_t)tid >> 4) * gridDim.x) * 16u + ((uint32_t)tid & 15u);
        const bool mine = (uint32_t)tid < nbu * 16u && my_row < rows;
        if (add && mine) {
            if (oldl) oldw = ll_load(oldl + my_row);
            else old = __ldcg(y + my_row);
        }
        float *pb = partial + pbuf * (kUnitBatch * kCWarps * 16);
        for (uint32_t j = 0; j < nbu; ++j) {
            const uint32_t u = u0 + j * gridDim.x;
            (void)u;
            float acc0 = 0.0f, acc1 = 0.0f;
            for (uint32_t s = 0; s < n_stages; ++s, ++n) {
                const uint32_t slot = n % P.n_slots, parity = (n / P.n_slots) & 1u;
                const bool ok = mbar_wait(&full[slot], parity, flags, P.spin_limit, P.status);
                    if (first_unit && s == 0) trace_stamp(P, oi, 4);
                const uint32_t base = smem_u32(slots + (size_t)slot * kSlotBytes);
                // This warp multiplies the chunk pair (2 warp, 2 warp + 1) of the stage.  Rows are dense in shared
                // memory (a multiple of 128 bytes apart), so rows g and g + 1 of one chunk would meet in the same
                // banks: even rows fetch the pair's first chunk while odd rows fetch its second, then the other
                // way round -- every 16-byte read of a quarter warp lands in its own bank group -- and each lane
                // keeps its own rows' two chunks apart again (no data moves between lanes).
                const uint32_t lc0 = 2u * (uint32_t)warp, par = (uint32_t)g & 1u;
                const uint32_t ch_a = s * kStageChunks + lc0;
                if (ok && ch_a < n_chunks) {
                    const uint32_t ra = base + (uint32_t)g * rs + (uint32_t)t4 * 16u, rb = ra + 8u * rs;
                    const uint32_t first = (lc0 + par) * kChunkCols, second = (lc0 + (par ^ 1u)) * kChunkCols;
                    int4 a1, a2, b1, b2;
                    uint32_t sa, sb;  // the pair's four block scales of rows g and g + 8 (8 bytes each, chunk-major)
                    asm volatile("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(a1.x), "=r"(a1.y), "=r"(a1.z), "=r"(a1.w) : "r"(ra + first));
                    asm volatile("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(b1.x), "=r"(b1.y), "=r"(b1.z), "=r"(b1.w) : "r"(rb + first));
                    asm volatile("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(a2.x), "=r"(a2.y), "=r"(a2.z), "=r"(a2.w) : "r"(ra + second));
                    asm volatile("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(b2.x), "=r"(b2.y), "=r"(b2.z), "=r"(b2.w) : "r"(rb + second));
                    const uint32_t soff = base + kQuantBytes + lc0 * 4u + (uint32_t)(t4 >> 1) * 2u;
                    {   // this lane's block (t4 / 2) of both chunks: two f16 scales 4 bytes apart, for each row
                        unsigned short s0, s1, s2, s3;
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s0) : "r"(soff + (uint32_t)g * kScaleStride));
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s1) : "r"(soff + 4u + (uint32_t)g * kScaleStride));
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s2) : "r"(soff + (uint32_t)(g + 8) * kScaleStride));
                        asm volatile("ld.shared.u16 %0, [%1];" : "=h"(s3) : "r"(soff + 4u + (uint32_t)(g + 8) * kScaleStride));
                        sa = (uint32_t)s0 | ((uint32_t)s1 << 16);
                        sb = (uint32_t)s2 | ((uint32_t)s3 << 16);
                    }
                    const bool two = ch_a + 1u < n_chunks;
                    const uint32_t c0 = ch_a * kChunkCols + (uint32_t)t4 * 16u;
                    int4 bx0 = make_int4(0, 0, 0, 0), bx1 = bx0;
                    if (b_live) {
                        bx0 = *(const int4 *)(xs + (size_t)(g & 3) * plane + c0);
                        if (two) bx1 = *(const int4 *)(xs + (size_t)(g & 3) * plane + c0 + kChunkCols);
                    }
                    const float2 cx0 = *(const float2 *)(coef_base + ((size_t)(c0 >> 5) * 4u + 2u * (t4 & 1)) * 4u);
                    const float2 cx1 = two ? *(const float2 *)(coef_base + ((size_t)((c0 + kChunkCols) >> 5) * 4u + 2u * (t4 & 1)) * 4u)
                                           : make_float2(0.f, 0.f);
                    // chunk h of the pair came with load `h == par ? first : second`
                    const int4 qa0 = par ? a2 : a1, qb0 = par ? b2 : b1, qa1 = par ? a1 : a2, qb1 = par ? b1 : b2;
                    int d0[4] = {0, 0, 0, 0}, d1[4] = {0, 0, 0, 0}, d2[4] = {0, 0, 0, 0}, d3[4] = {0, 0, 0, 0};
                    mma_s8(d0, qa0.x, qb0.x, qa0.y, qb0.y, bx0.x, bx0.y);
                    mma_s8(d1, qa0.z, qb0.z, qa0.w, qb0.w, bx0.z, bx0.w);
                    mma_s8(d2, qa1.x, qb1.x, qa1.y, qb1.y, bx1.x, bx1.y);
                    mma_s8(d3, qa1.z, qb1.z, qa1.w, qb1.w, bx1.z, bx1.w);
                    const float va0 = fmaf((float)(d0[1] + d1[1]), cx0.y, (float)(d0[0] + d1[0]) * cx0.x);
                    const float vb0 = fmaf((float)(d0[3] + d1[3]), cx0.y, (float)(d0[2] + d1[2]) * cx0.x);
                    const float va1 = fmaf((float)(d2[1] + d3[1]), cx1.y, (float)(d2[0] + d3[0]) * cx1.x);
                    const float vb1 = fmaf((float)(d2[3] + d3[3]), cx1.y, (float)(d2[2] + d3[2]) * cx1.x);
                    const float2 fa = __half22float2(*(const __half2 *)&sa), fb = __half22float2(*(const __half2 *)&sb);
                    acc0 = fmaf(fa.x, va0, acc0);
                    acc1 = fmaf(fb.x, vb0, acc1);
                    if (two) {  // past the last chunk the scale bytes are whatever the slot held before
                        acc0 = fmaf(fa.y, va1, acc0);
                        acc1 = fmaf(fb.y, vb1, acc1);
                    }
                }
                __syncwarp();
                if (lane == 0) mbar_arrive(&empty[slot]);  // this warp is done with the stage (one arrival per warp frees it)
            }
            if (first_unit) trace_stamp(P, oi, 5);
            first_unit = false;
            acc0 += __shfl_xor_sync(0xffffffffu, acc0, 1);
            acc0 += __shfl_xor_sync(0xffffffffu, acc0, 2);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 1);
            acc1 += __shfl_xor_sync(0xffffffffu, acc1, 2);
            if (t4 == 0) {
                pb[(j * kCWarps + warp) * 16 + g] = acc0;
                pb[(j * kCWarps + warp) * 16 + g + 8] = acc1;
            }
        }
        consumer_sync();
        if (mine) {
            float v = 0.0f;
#pragma unroll
            for (int w = 0; w < kCWarps; ++w) v += pb[(((uint32_t)tid >> 4) * kCWarps + w) * 16 + (tid & 15)];
            if (add) {
                if (oldl) {
                    uint32_t spin = 0;
                    while ((uint32_t)(oldw >> 32) != old_seq && poll_again(P, flags, spin)) oldw = ll_load(oldl + my_row);
                    old = __uint_as_float((uint32_t)oldw);
                }
                v = old + v;
            }
            if (!flags[0]) {  // a stopping CTA publishes nothing: its consumers must not take a wrong value
                ll_store(yl + my_row, v, seq);
                if (plain) y[my_row] = v;
            }
        }
        if (u0 == u_first) trace_stamp(P, oi, 6);
        pbuf ^= 1u;  // the next batch writes the other buffer; its sync orders this one's readers
    }
}

// ---- weight producer -------------------------------------------------------------------
// This CTA's weight stages in program order: (operator, unit, stage of the unit).
struct stage_cursor {
    uint32_t oi, u, s, count;  // count: stages before this one
    uint32_t rows, cols, n_units, n_stages;
    const step_op *op;
    __device__ bool seek(const step_params &P) {  // position on the first unit of operator `oi` or a later one
        for (; oi < P.n_ops; ++oi) {
            op = P.ops + oi;
            if (op->kind != STEP_GEMV) continue;
            rows = op->rows;
            cols = op->cols;
            n_units = (rows + 15u) / 16u;
            n_stages = (cols / kChunkCols + kStageChunks - 1u) / kStageChunks;
            u = (blockIdx.x + gridDim.x - op->first_cta) % gridDim.x;
            s = 0;
            if (u < n_units) return true;
        }
        return false;
    }
    __device__ bool next(const step_params &P) {
        ++count;
        if (++s < n_stages) return true;
        s = 0;
        u += gridDim.x;
        if (u < n_units) return true;
        ++oi;
        return seek(P);
    }
};

// Stages run through two cursors: the far one asks L2 for a stage (tensor-map prefetch, no shared
// memory involved) `l2_ahead` stages before the near one copies it into the ring.  The ring alone
// (ten stages) covers about four microseconds of the HBM stream; while the consumers stage
// activations or run attention it fills up and the stream would stop -- L2 keeps it going.
// Returns the number of stages requested into the ring.
__device__ __forceinline__ uint32_t producer_loop(const step_params &P, unsigned char *slots, uint64_t *full, uint64_t *empty,
                                  volatile uint32_t *flags) {
    const int lane = threadIdx.x & 31;
    stage_cursor near = {}, far = {};
    bool near_ok = near.seek(P), far_ok = far.seek(P);
    uint32_t traced = 0xFFFFFFFFu;
    while (near_ok && !flags[0]) {
        while (far_ok && far.count < near.count + P.l2_ahead) {
            const uint32_t ch0 = far.s * kStageChunks;
            if (lane == 0)
                asm volatile("cp.async.bulk.prefetch.tensor.2d.L2.global [%0, {%1, %2}];" ::"l"(far.op->wmap),
                             "r"((int)(ch0 * (kChunkCols / 4u))), "r"((int)(far.u * 16u))
                             : "memory");
            else if ((uint32_t)lane <= 16u && far.u * 16u + (uint32_t)lane - 1u < far.rows)  // the rows' block scales
                asm volatile("prefetch.global.L2 [%0];" ::"l"((const unsigned char *)far.op->p[1] +
                                                               ((size_t)(far.u * 16u + (uint32_t)lane - 1u) * (far.cols / 32u) +
                                                                (size_t)ch0 * 2u) * 2u));
            far_ok = far.next(P);
        }
        const step_op &op = *near.op;
        const uint32_t n = near.count, u = near.u, cols = near.cols, nb = cols / 32u;
        const uint32_t n_chunks = cols / kChunkCols;
        const unsigned char *d = (const unsigned char *)op.p[1];
        const uint32_t unit_rows = min(16u, near.rows - u * 16u);
        const uint32_t slot = n % P.n_slots, parity = ((n / P.n_slots) & 1u) ^ 1u;
        // the slot's previous tenant has been read by every consumer warp
        if (!mbar_wait(&empty[slot], parity, flags, P.spin_limit, P.status)) return n;
        if (P.trace != nullptr && blockIdx.x == 0 && lane == 0 && traced != near.oi) {  // when the operator's first stage was requested
            u64 t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            P.trace[(size_t)near.oi * 8 + 7] = t;
            traced = near.oi;
        }
        const uint32_t ch0 = near.s * kStageChunks, nch = min(kStageChunks, n_chunks - ch0);
        unsigned char *dst = slots + (size_t)slot * kSlotBytes;
        if (lane == 0) {
            // the whole box arrives (columns and rows past the matrix as zeros), so the stage's
            // byte count does not depend on where it sits
            mbar_expect_tx(&full[slot], 16u * op.row_stride);
            asm volatile(
                "cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%3, %4}], [%2];" ::"r"(
                    smem_u32(dst)),
                "l"(op.wmap), "r"(smem_u32(&full[slot])), "r"((int)(ch0 * (kChunkCols / 4u))), "r"((int)(u * 16u))
                : "memory");
        }
        // block scales of the stage: nch * 4 bytes per row; lane l takes row l / 2 and every other piece
        // of it, in the widest copies the row's alignment allows (a row starts cols / 16 bytes after the
        // one before it)
        {
            const uint32_t r = (uint32_t)lane >> 1, half = (uint32_t)lane & 1u;
            if (r < unit_rows) {
                const unsigned char *src = d + ((size_t)(u * 16u + r) * nb + (size_t)ch0 * 2u) * 2u;
                const uint32_t to = smem_u32(dst + kQuantBytes + r * kScaleStride), bytes = nch * 4u;
                if ((cols & 255u) == 0u) {
                    for (uint32_t o = half * 16u; o < bytes; o += 32u)
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 16;" ::"r"(to + o), "l"(src + o) : "memory");
                } else if ((cols & 127u) == 0u) {
                    for (uint32_t o = half * 8u; o < bytes; o += 16u)
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 8;" ::"r"(to + o), "l"(src + o) : "memory");
                } else {
                    for (uint32_t o = half * 4u; o < bytes; o += 8u)
                        asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(to + o), "l"(src + o) : "memory");
                }
            }
        }
        asm volatile("cp.async.mbarrier.arrive.noinc.shared::cta.b64 [%0];" ::"r"(smem_u32(&full[slot])) : "memory");
        near_ok = near.next(P);
    }
    return near.count;
}

// The producer leaves only after everything it requested has landed (a CTA must not retire with
// copies in flight to its shared memory): it waits, bounded, for the last stages it requested.  When
// the consumers took them all this returns at once (a completed phase stays completed).
__device__ __forceinline__ void producer_drain(const step_params &P, uint64_t *full, uint32_t issued) {
    const uint32_t from = issued > P.n_slots ? issued - P.n_slots : 0u;
    for (uint32_t m = from; m < issued; ++m) {
        const uint32_t addr = smem_u32(&full[m % P.n_slots]), parity = (m / P.n_slots) & 1u;
        for (uint32_t spin = 0; spin < P.spin_limit; ++spin)
            if (mbar_try(addr, parity)) break;
    }
}

// ---- attention item --------------------------------------------------------------------
__device__ __forceinline__ uint32_t attn_start(uint32_t seq, uint32_t window) {
    return window != 0u && seq > window ? seq - window : 0u;
}

template <int G, int HD>
struct attn_shared {
    static constexpr int PAIRS = HD / 2;
    static constexpr int KP = 128 / PAIRS > 0 ? 128 / PAIRS : 1;
    float qs[G][HD];
    __half kh[HD];
    __half vh[HD];
    float sc[G][kAttnSplit];
    float stat[G][2];
    float opart[KP][G][HD];
};

// One (KV head, 64-key split) item by 128 threads: q/k RMS norm, RoPE, f16 KV store (the split that
// holds the new position), scores, split softmax, values.  The arithmetic and the merge order are
// those of attention_decode_fast_kernel (tm_cuda_ops.cu), so both give the same bits; the splits'
// partial results travel as flagged words and the group of the newest split merges them.
template <int G, int HD>
__device__ __forceinline__ void attn_item(const step_params &P, const step_op &op, uint32_t oi, uint32_t pos, uint32_t kvh,
                          uint32_t split, int tid, unsigned char *sm, int bar_id, volatile uint32_t *flags) {
    using S = attn_shared<G, HD>;
    static_assert(sizeof(S) <= kAttnSub, "attention group shared memory");
    constexpr int EPL = HD / 32, PAIRS = S::PAIRS, KP = S::KP;
    constexpr int KEYS = kAttnSplit / KP;
    S &s = *(S *)sm;
    const int lane = tid & 31, warp = tid >> 5;
    const float *q = (const float *)op.p[0], *k = (const float *)op.p[1], *v = (const float *)op.p[2];
    const float *q_norm = (const float *)op.p[3], *k_norm = (const float *)op.p[4], *inv_freq = (const float *)op.p[5];
    __half *kc = (__half *)op.p[6], *vc = (__half *)op.p[7];
    float *out = (float *)op.p[8];
    const uint32_t cap = op.u[3], window = op.u[4];
    const float eps = op.eps, scale = op.scale;
    const uint32_t nsplit = (cap + kAttnSplit - 1) / kAttnSplit;
    const __half *kp = kc + (size_t)kvh * cap * HD, *vp = vc + (size_t)kvh * cap * HD;
    const uint32_t seq = pos + 1u, start = attn_start(seq, window);
    const uint32_t first = start / kAttnSplit, last = pos / kAttnSplit;
    const bool owns_new = split == last;
    const uint32_t my_seq = P.seq_base + oi;
    // this thread's half of key row split*64 + tid/2 (rows of earlier steps: earlier launches wrote them)
    constexpr int NL = HD / 16;
    int4 kraw[NL];
    {
        const uint32_t j = min(split * kAttnSplit + ((uint32_t)tid >> 1), cap - 1u);
        const __half *kr = kp + (size_t)j * HD + (tid & 1) * (HD / 2);
#pragma unroll
        for (int c = 0; c < NL; ++c) kraw[c] = *(const int4 *)(kr + c * 8);
    }
    // ---- q_0..q_{G-1} (and k for the owning split): RMS norm + RoPE, one warp each ----
    for (int vec = warp; vec < G + (owns_new ? 1 : 0); vec += 4) {
        const bool is_k = vec == G;
        const size_t off = is_k ? (size_t)kvh * HD : ((size_t)kvh * G + vec) * HD;
        const float *src = (is_k ? k : q) + off;
        const u64 *srcl = is_k ? op.in[1] : op.in[0];
        const uint32_t src_seq = P.seq_base + (is_k ? op.in_op[1] : op.in_op[0]) + P.seq_skew;
        const float *nw = is_k ? k_norm : q_norm;
        float x[EPL], w[EPL], vnew[EPL];
#pragma unroll
        for (int r = 0; r < EPL; ++r) w[r] = __ldg(nw + lane + 32 * r);
        if (srcl) {
            u64 xw[EPL], vw[EPL];
#pragma unroll
            for (int r = 0; r < EPL; ++r) {
                xw[r] = ll_load(srcl + off + lane + 32 * r);
                vw[r] = is_k && op.in[2] ? ll_load(op.in[2] + off + lane + 32 * r) : 0;
            }
            const uint32_t v_seq = P.seq_base + op.in_op[2] + P.seq_skew;
            uint32_t spin = 0;
            for (;;) {
                bool again = false;
#pragma unroll
                for (int r = 0; r < EPL; ++r) {
                    if ((uint32_t)(xw[r] >> 32) != src_seq) { xw[r] = ll_load(srcl + off + lane + 32 * r); again = true; }
                    if (is_k && op.in[2] && (uint32_t)(vw[r] >> 32) != v_seq) {
                        vw[r] = ll_load(op.in[2] + off + lane + 32 * r);
                        again = true;
                    }
                }
                if (!again || !poll_again(P, flags, spin)) break;
            }
#pragma unroll
            for (int r = 0; r < EPL; ++r) {
                x[r] = __uint_as_float((uint32_t)xw[r]);
                vnew[r] = is_k ? (op.in[2] ? __uint_as_float((uint32_t)vw[r]) : __ldcg(v + off + lane + 32 * r)) : 0.0f;
            }
        } else {
#pragma unroll
            for (int r = 0; r < EPL; ++r) {
                x[r] = __ldcg(src + lane + 32 * r);
                vnew[r] = is_k ? __ldcg(v + off + lane + 32 * r) : 0.0f;
            }
        }
        float ss = 0.0f;
#pragma unroll
        for (int r = 0; r < EPL; ++r) ss = fmaf(x[r], x[r], ss);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, o);
        const float inv = 1.0f / sqrtf(ss / (float)HD + eps);
#pragma unroll
        for (int r = 0; r < EPL; ++r) x[r] = x[r] * inv * w[r];
#pragma unroll
        for (int r = 0; r < EPL / 2; ++r) {
            float sn, cs;
            sincosf((float)pos * __ldg(inv_freq + lane + 32 * r), &sn, &cs);
            const float a0 = x[r], b0 = x[r + EPL / 2];
            x[r] = a0 * cs - b0 * sn;
            x[r + EPL / 2] = a0 * sn + b0 * cs;
        }
        if (is_k) {
#pragma unroll
            for (int r = 0; r < EPL; ++r) {
                const uint32_t e = lane + 32 * r;
                const __half hk = __float2half_rn(x[r]), hv = __float2half_rn(vnew[r]);
                s.kh[e] = hk;
                s.vh[e] = hv;
                if (!flags[0]) {
                    kc[((size_t)kvh * cap + pos) * HD + e] = hk;
                    vc[((size_t)kvh * cap + pos) * HD + e] = hv;
                }
            }
        } else {
#pragma unroll
            for (int r = 0; r < EPL; ++r) s.qs[vec][lane + 32 * r] = x[r];
        }
    }
    group_sync(bar_id);
    // ---- scores: two threads per key, half the dims each ----
    {
        const uint32_t jj = tid >> 1, hsel = tid & 1, j = split * kAttnSplit + jj;
        const bool valid = j >= start && j < seq;
        float dot[G][2];
#pragma unroll
        for (int g = 0; g < G; ++g) dot[g][0] = dot[g][1] = 0.0f;
        if (valid) {
            int4 raw[NL];
            const bool fresh = owns_new && j == pos;
#pragma unroll
            for (int c = 0; c < NL; ++c) raw[c] = fresh ? *(const int4 *)(s.kh + hsel * (HD / 2) + c * 8) : kraw[c];
#pragma unroll
            for (int c = 0; c < NL; ++c) {
                const __half2 *h2 = (const __half2 *)&raw[c];
                float kf[8];
#pragma unroll
                for (int e = 0; e < 4; ++e) {
                    const float2 f = __half22float2(h2[e]);
                    kf[2 * e] = f.x;
                    kf[2 * e + 1] = f.y;
                }
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float *qp = &s.qs[g][hsel * (HD / 2) + c * 8];
                    const float4 q0 = *(const float4 *)qp, q1 = *(const float4 *)(qp + 4);
                    float t = dot[g][c & 1];
                    t = fmaf(q0.x, kf[0], t); t = fmaf(q0.y, kf[1], t); t = fmaf(q0.z, kf[2], t); t = fmaf(q0.w, kf[3], t);
                    t = fmaf(q1.x, kf[4], t); t = fmaf(q1.y, kf[5], t); t = fmaf(q1.z, kf[6], t); t = fmaf(q1.w, kf[7], t);
                    dot[g][c & 1] = t;
                }
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            float d = dot[g][0] + dot[g][1];
            d += __shfl_xor_sync(0xffffffffu, d, 1);
            if (hsel == 0) s.sc[g][jj] = valid ? d * scale : -INFINITY;
        }
    }
    group_sync(bar_id);
    // ---- split softmax: warp g owns head g ----
    for (int g = warp; g < G; g += 4) {
        const float s0 = s.sc[g][lane], s1 = s.sc[g][lane + 32];
        float mx = fmaxf(s0, s1);
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, o));
        const float p0 = s0 == -INFINITY ? 0.0f : expf(s0 - mx), p1 = s1 == -INFINITY ? 0.0f : expf(s1 - mx);
        float sum = p0 + p1;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) sum += __shfl_xor_sync(0xffffffffu, sum, o);
        s.sc[g][lane] = p0;
        s.sc[g][lane + 32] = p1;
        if (lane == 0) {
            s.stat[g][0] = mx;
            s.stat[g][1] = sum;
        }
    }
    group_sync(bar_id);
    // ---- values: thread = (dim pair, key part); keys of a part in order ----
    {
        const uint32_t kpart = tid / PAIRS < KP ? tid / PAIRS : 0, dp0 = tid % PAIRS;
        const uint32_t jbase = split * kAttnSplit + kpart * KEYS;
        float acc[G][2];
#pragma unroll
        for (int g = 0; g < G; ++g) acc[g][0] = acc[g][1] = 0.0f;
#pragma unroll 1
        for (int kb = 0; kb < KEYS; kb += 8) {
            __half2 vv[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const uint32_t j = jbase + kb + c;
                const uint32_t jc = j < seq ? j : pos;  // rows past the sequence carry weight 0
                const __half *vr = owns_new && jc == pos ? s.vh : vp + (size_t)min(jc, cap - 1u) * HD;
                vv[c] = j < seq ? *(const __half2 *)(vr + 2 * dp0) : __float2half2_rn(0.0f);
            }
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float2 f = __half22float2(vv[c]);
#pragma unroll
                for (int g = 0; g < G; ++g) {
                    const float pj = s.sc[g][kpart * KEYS + kb + c];
                    acc[g][0] = fmaf(pj, f.x, acc[g][0]);
                    acc[g][1] = fmaf(pj, f.y, acc[g][1]);
                }
            }
        }
#pragma unroll
        for (int g = 0; g < G; ++g) {
            s.opart[kpart][g][2 * dp0] = acc[g][0];
            s.opart[kpart][g][2 * dp0 + 1] = acc[g][1];
        }
    }
    group_sync(bar_id);
    // ---- this split's (m, l, o): finish here when it is the only one, else publish it; the group
    // of the newest split then merges all of them in split order ----
    const bool single = first == last;
    constexpr uint32_t stride = HD + 2;
    u64 *part = P.attn_ll + ((size_t)kvh * nsplit + split) * G * stride;
    const bool quiet = flags[0] != 0u;
    for (uint32_t i = tid; i < G * HD; i += 128) {
        const uint32_t g = i / HD, d = i % HD;
        float o = 0.0f;
#pragma unroll
        for (int kq = 0; kq < KP; ++kq) o += s.opart[kq][g][d];
        if (single) {
            const float r = o / s.stat[g][1];
            if (!quiet) {
                ll_store(op.out + ((size_t)kvh * G + g) * HD + d, r, my_seq);
                if (op.write_plain) out[((size_t)kvh * G + g) * HD + d] = r;
            }
        } else if (!owns_new && !quiet) {
            ll_store(part + g * stride + 2 + d, o, my_seq);
        }
    }
    if (!single && !owns_new && tid < G && !quiet) {
        ll_store(part + tid * stride, s.stat[tid][0], my_seq);
        ll_store(part + tid * stride + 1, s.stat[tid][1], my_seq);
    }
    if (single || !owns_new) {
        group_sync(bar_id);  // the group's shared memory is free for its next item
        return;
    }
    // merge: one thread per (head, dim); the partials of 4 splits are polled together
    for (uint32_t i = tid; i < G * HD; i += 128) {
        const uint32_t g = i / HD, d = i % HD;
        const u64 *base = P.attn_ll + ((size_t)kvh * nsplit + first) * G * stride + g * stride;
        const uint32_t nact = last - first + 1;
        float own_o = 0.0f;
#pragma unroll
        for (int kq = 0; kq < KP; ++kq) own_o += s.opart[kq][g][d];
        float M = -INFINITY, L = 0.0f, O = 0.0f;
        for (uint32_t s0 = 0; s0 < nact; s0 += 4) {
            float mb[4], lb[4], ob[4];
            u64 mw[4], lw[4], ow[4];
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t sp = s0 + c < nact ? s0 + c : nact - 1;
                const u64 *pb = base + (size_t)sp * G * stride;
                const bool mine = sp == nact - 1;  // this group's own split: from shared memory
                mw[c] = mine ? 0 : ll_load(pb);
                lw[c] = mine ? 0 : ll_load(pb + 1);
                ow[c] = mine ? 0 : ll_load(pb + 2 + d);
            }
            uint32_t spin = 0;
            for (;;) {
                bool again = false;
#pragma unroll
                for (int c = 0; c < 4; ++c) {
                    const uint32_t sp = s0 + c < nact ? s0 + c : nact - 1;
                    if (sp == nact - 1) continue;
                    const u64 *pb = base + (size_t)sp * G * stride;
                    if ((uint32_t)(mw[c] >> 32) != my_seq) { mw[c] = ll_load(pb); again = true; }
                    if ((uint32_t)(lw[c] >> 32) != my_seq) { lw[c] = ll_load(pb + 1); again = true; }
                    if ((uint32_t)(ow[c] >> 32) != my_seq) { ow[c] = ll_load(pb + 2 + d); again = true; }
                }
                if (!again || !poll_again(P, flags, spin)) break;
            }
#pragma unroll
            for (int c = 0; c < 4; ++c) {
                const uint32_t sp = s0 + c < nact ? s0 + c : nact - 1;
                const bool mine = sp == nact - 1;
                mb[c] = mine ? s.stat[g][0] : __uint_as_float((uint32_t)mw[c]);
                lb[c] = mine ? s.stat[g][1] : __uint_as_float((uint32_t)lw[c]);
                ob[c] = mine ? own_o : __uint_as_float((uint32_t)ow[c]);
            }
            float mx = M;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (s0 + c < nact) mx = fmaxf(mx, mb[c]);
            const float a = expf(M - mx);
            L *= a;
            O *= a;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                if (s0 + c < nact) {
                    const float wgt = expf(mb[c] - mx);
                    L = fmaf(wgt, lb[c], L);
                    O = fmaf(wgt, ob[c], O);
                }
            M = mx;
        }
        if (!flags[0]) {
            const float r = O / L;
            ll_store(op.out + ((size_t)kvh * G + g) * HD + d, r, my_seq);
            if (op.write_plain) out[((size_t)kvh * G + g) * HD + d] = r;
        }
    }
    group_sync(bar_id);
}

template <int G, int HD>
__device__ __forceinline__ void attn_consume(const step_params &P, const step_op &op, uint32_t oi, uint32_t pos, unsigned char *xs,
                             volatile uint32_t *flags) {
    const int tid = threadIdx.x & 127, sub = threadIdx.x >> 7;
    const uint32_t kv_heads = op.u[1], window = op.u[4];
    const uint32_t seq = pos + 1u, start = attn_start(seq, window);
    const uint32_t first = start / kAttnSplit, last = pos / kAttnSplit, nact = last - first + 1u;
    const uint32_t items = kv_heads * nact;
    // Items dealt over the CTAs first, then over the two warp groups of a CTA.  The newest split of
    // every KV head (the merging one, which waits for the others) comes LAST in the order: a group works
    // through its items one after the other, so nothing a merger waits for can be queued behind it.
    const uint32_t plain_items = kv_heads * (nact - 1u);
    for (uint32_t it = blockIdx.x + gridDim.x * (uint32_t)sub; it < items; it += gridDim.x * (kCThreads / 128u)) {
        uint32_t kvh, split;
        if (it >= plain_items) {
            kvh = it - plain_items;
            split = last;
        } else {
            kvh = it / (nact - 1u);
            split = first + it % (nact - 1u);
        }
        attn_item<G, HD>(P, op, oi, pos, kvh, split, tid, xs + (size_t)sub * kAttnSub, 2 + sub, flags);
    }
}

__device__ __forceinline__ bool better(float av, uint32_t ai, float bv, uint32_t bi) {
    if (ai == kArgmaxNone) return false;
    if (bi == kArgmaxNone) return true;
    return av > bv || (av == bv && ai < bi);
}

// Greedy rule over the consumer threads' candidates (crates/backend/src/sampling.rs:68-82: NaN
// skipped, larger wins, ties to the lower index); thread 0 returns the CTA's winner.
__device__ __forceinline__ void argmax_cta(float &v, uint32_t &i, float *red) {
    uint32_t *ri = (uint32_t *)red + 16;
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) {
        const float ov = __shfl_down_sync(0xffffffffu, v, o);
        const uint32_t oi = __shfl_down_sync(0xffffffffu, i, o);
        if (better(ov, oi, v, i)) { v = ov; i = oi; }
    }
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    if (lane == 0) { red[warp] = v; ri[warp] = i; }
    consumer_sync();
    if (warp == 0) {
        v = lane < kCWarps ? red[lane] : -INFINITY;
        i = lane < kCWarps ? ri[lane] : kArgmaxNone;
#pragma unroll
        for (int o = 16; o > 0; o >>= 1) {
            const float ov = __shfl_down_sync(0xffffffffu, v, o);
            const uint32_t oi = __shfl_down_sync(0xffffffffu, i, o);
            if (better(ov, oi, v, i)) { v = ov; i = oi; }
        }
    }
    consumer_sync();
}

__global__ void __launch_bounds__(kStepThreads, 1) decode_step_kernel(const step_params P) {
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *xs = smem;
    unsigned char *slots = smem + P.xs_bytes;
    uint64_t *full = (uint64_t *)(slots + (size_t)P.n_slots * kSlotBytes);
    uint64_t *empty = full + kMaxSlots;
    float *partial = (float *)(empty + kMaxSlots);
    float *red = partial + 2 * kUnitBatch * kCWarps * 16;
    uint32_t *desc = (uint32_t *)(red + 32);                 // two operator descriptors, used in turn
    volatile uint32_t *flags = (volatile uint32_t *)(desc + 2 * kDescWords);
    {   // a program whose earlier launch gave up a wait stays stopped: its flagged words are no longer whole
        uint32_t st;
        asm volatile("ld.relaxed.gpu.global.u32 %0, [%1];" : "=r"(st) : "l"(P.status) : "memory");
        if (st) return;
    }
    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < P.n_slots; ++s) {
            mbar_init(&full[s], 33);   // lane 0's expect_tx arrival + the 32 producer lanes' copy arrivals
            mbar_init(&empty[s], kCWarps);
        }
        flags[0] = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (threadIdx.x < kDescWords) desc[threadIdx.x] = ((const uint32_t *)P.ops)[threadIdx.x];
    __syncthreads();
    if (threadIdx.x >= kCThreads) {
        const uint32_t issued = producer_loop(P, slots, full, empty, flags);
        producer_drain(P, full, issued);
        return;
    }
    uint32_t n = 0, pbuf = 0;
    const bool tracing = P.trace != nullptr && blockIdx.x == 0 && threadIdx.x == 0;
    auto stamp = [&](uint32_t oi, int k) {
        if (tracing) {
            u64 t;
            asm volatile("mov.u64 %0, %%globaltimer;" : "=l"(t));
            P.trace[(size_t)oi * 8 + k] = t;
        }
    };
    for (uint32_t oi = 0; oi < P.n_ops; ++oi) {
        // the next operator's descriptor travels to shared memory while this one runs
        if (oi + 1 < P.n_ops && threadIdx.x < kDescWords)
            desc[((oi + 1) & 1u) * kDescWords + threadIdx.x] = ((const uint32_t *)(P.ops + oi + 1))[threadIdx.x];
        const step_op &op = *(const step_op *)(desc + (oi & 1u) * kDescWords);
        const uint32_t seq = P.seq_base + oi;
        stamp(oi, 0);
        switch (op.kind) {
            case STEP_GEMV:
                stage_activations(P, op, oi, xs, red, flags);
                stamp(oi, 1);
                gemv_consume(P, op, oi, xs, slots, full, empty, partial, flags, n, pbuf);
                break;
            case STEP_EMBED:
                if (blockIdx.x == 0) {
                    const signed char *q = (const signed char *)op.p[0];
                    const __half *d = (const __half *)op.p[1];
                    const uint32_t *ids = (const uint32_t *)op.p[2], *pos = (const uint32_t *)op.p[3];
                    float *out = (float *)op.p[4];
                    uint32_t slot = op.u[0];
                    if (pos) slot = slot + __ldcg(pos) + op.u[1];
                    long row = -1;
                    if (slot < op.u[2]) {
                        const uint32_t id = __ldcg(ids + slot);
                        if (id < op.rows) row = (long)id;
                    }
                    const uint32_t nb = op.cols / 32u;
                    for (uint32_t c = threadIdx.x; c < op.cols; c += kCThreads) {
                        float v = 0.0f;
                        if (row >= 0) {
                            v = __half2float(d[(size_t)row * nb + c / 32u]) * (float)q[(size_t)row * op.cols + c];
                            if (op.scale != 0.0f) v *= op.scale;
                        }
                        ll_store(op.out + c, v, seq);
                        if (op.write_plain) out[c] = v;
                    }
                }
                break;
            case STEP_ATTN: {
                const uint32_t pos = __ldcg((const uint32_t *)op.p[10]);
                if (pos >= op.u[3]) {  // past the cache: tell the host; consumers of the output will give up
                    if (blockIdx.x == 0 && threadIdx.x == 0) atomicOr((uint32_t *)op.p[11], 1u);
                    break;
                }
                const uint32_t g = op.u[0] / op.u[1], hd = op.u[2];
                if (hd == 128) {
                    if (g == 1) attn_consume<1, 128>(P, op, oi, pos, xs, flags);
                    else if (g == 2) attn_consume<2, 128>(P, op, oi, pos, xs, flags);
                    else attn_consume<4, 128>(P, op, oi, pos, xs, flags);
                } else {
                    if (g == 1) attn_consume<1, 256>(P, op, oi, pos, xs, flags);
                    else if (g == 2) attn_consume<2, 256>(P, op, oi, pos, xs, flags);
                    else attn_consume<4, 256>(P, op, oi, pos, xs, flags);
                }
                break;
            }
            case STEP_NORM_ADD:
                if (blockIdx.x == 0) {  // x += rmsnorm(p) * w, one row: p is polled once, then re-read
                    const float *pp = (const float *)op.p[0], *w = (const float *)op.p[1];
                    float *x = (float *)op.p[2];
                    const uint32_t pseq = P.seq_base + op.in_op[0] + P.seq_skew, xseq = P.seq_base + op.in_op[1] + P.seq_skew;
                    float sq = 0.0f;
                    for (uint32_t c = threadIdx.x; c < op.cols; c += kCThreads) {
                        const float pv = op.in[0] ? ll_wait(P, op.in[0] + c, pseq, flags) : __ldcg(pp + c);
                        sq = fmaf(pv, pv, sq);
                    }
#pragma unroll
                    for (int o = 16; o > 0; o >>= 1) sq += __shfl_xor_sync(0xffffffffu, sq, o);
                    if ((threadIdx.x & 31) == 0) red[threadIdx.x >> 5] = sq;
                    consumer_sync();
                    float t = 0.0f;
#pragma unroll
                    for (int k = 0; k < kCWarps; ++k) t += red[k];
                    const float inv = 1.0f / sqrtf(t / (float)op.cols + op.eps);
                    for (uint32_t c = threadIdx.x; c < op.cols; c += kCThreads) {
                        const float pv = op.in[0] ? ll_wait(P, op.in[0] + c, pseq, flags) : __ldcg(pp + c);
                        const float xv = op.in[1] ? ll_wait(P, op.in[1] + c, xseq, flags) : __ldcg(x + c);
                        if (!flags[0]) {
                            const float r = __fadd_rn(xv, __fmul_rn(__fmul_rn(pv, inv), __ldg(w + c)));
                            ll_store(op.out + c, r, seq);
                            if (op.write_plain) x[c] = r;
                        }
                    }
                }
                break;
            case STEP_ARGMAX: {
                const float *x = (const float *)op.p[0];
                const uint32_t nx = op.u[0], xseq = P.seq_base + op.in_op[0] + P.seq_skew;
                float v = -INFINITY;
                uint32_t i = kArgmaxNone;
                for (uint32_t k = blockIdx.x * kCThreads + threadIdx.x; k < nx; k += gridDim.x * kCThreads) {
                    const float xv = op.in[0] ? ll_wait(P, op.in[0] + k, xseq, flags) : __ldcg(x + k);
                    if (!isnan(xv) && better(xv, k, v, i)) { v = xv; i = k; }
                }
                argmax_cta(v, i, red);
                if (threadIdx.x == 0 && !flags[0]) {
                    ll_store(P.argmax_ll + 2 * blockIdx.x, v, seq);
                    ll_store_u32(P.argmax_ll + 2 * blockIdx.x + 1, i, seq);
                }
                if (blockIdx.x == 0) {
                    v = -INFINITY;
                    i = kArgmaxNone;
                    for (uint32_t k = threadIdx.x; k < gridDim.x; k += kCThreads) {
                        const float cv = ll_wait(P, P.argmax_ll + 2 * k, seq, flags);
                        const uint32_t ci = __float_as_uint(ll_wait(P, P.argmax_ll + 2 * k + 1, seq, flags));
                        if (better(cv, ci, v, i)) { v = cv; i = ci; }
                    }
                    argmax_cta(v, i, red);
                    if (threadIdx.x == 0 && !flags[0]) {
                        const uint32_t *pos = (const uint32_t *)op.p[2];
                        const uint32_t slot = pos ? op.u[1] + __ldcg(pos) : op.u[1];
                        if (slot < op.u[2]) {
                            ((uint32_t *)op.p[1])[slot] = i;
                            if (op.p[3]) ((uint32_t *)op.p[3])[slot] = i;
                        }
                    }
                }
                break;
            }
            case STEP_POS_ADD: {
                // The counter may move only when no CTA will read it again: every CTA counts itself in
                // when it gets here (all its earlier operators are done), CTA 0 waits for all of them.
                consumer_sync();
                if (threadIdx.x == 0) {
                    __threadfence();
                    atomicAdd(P.arrivals, 1u);
                    if (blockIdx.x == 0) {
                        const uint32_t target = P.arrivals_base + (op.u[1] + 1u) * gridDim.x;
                        uint32_t spin = 0;
                        for (;;) {
                            uint32_t a;
                            asm volatile("ld.acquire.gpu.global.u32 %0, [%1];" : "=r"(a) : "l"(P.arrivals) : "memory");
                            if ((int32_t)(a - target) >= 0) break;
                            if (!poll_again(P, flags, spin)) break;
                        }
                        if (!flags[0]) {
                            uint32_t *c = (uint32_t *)op.p[0];
                            *c = __ldcg(c) + op.u[0];
                        }
                    }
                }
                break;
            }
            default: break;
        }
        stamp(oi, 2);
        consumer_sync();  // the next descriptor is in place; shared memory of this operator is free
    }
}

}  // namespace

// ---- host side: recording and launching -------------------------------------------------
struct tm_step_program {
    std::vector<step_op> ops;
    std::vector<uint32_t> out_len;  // floats each operator writes (0: none)
    unsigned char *dev = nullptr;   // [ops | arrivals, status | argmax words | tensor maps | flagged vectors | attention partials]
    size_t dev_bytes = 0, ops_bytes = 0, maps_off = 0, ll_off = 0, attn_off = 0;
    uint32_t max_ops = 0, pos_adds = 0;
    uint64_t ll_words = 0, attn_words = 0;  // capacity asked for at begin_program
    uint64_t launches = 0;
    uint32_t xs_bytes = 0, n_slots = 0, smem = 0;
    uint32_t next_cta = 0;          // the round-robin deal of units continues across operators
    uint32_t seq_skew = 0, spin_limit = 1u << 18, l2_ahead = 0;
    u64 *trace = nullptr;           // device, [ops][8], allocated on the first trace request
    int grid = 0;
};

static size_t program_bytes(uint32_t max_ops, uint64_t ll_words, uint64_t attn_words) {
    return tm_round_up((size_t)max_ops * sizeof(step_op), 256) + 256 + 2 * 8 * 1024 + (size_t)max_ops * 128 +
           tm_round_up((size_t)ll_words * 8, 256) + tm_round_up((size_t)attn_words * 8, 256);
}

typedef CUresult (*encode_tiled_fn)(CUtensorMap *, CUtensorMapDataType, cuuint32_t, void *, const cuuint64_t *,
                                    const cuuint64_t *, const cuuint32_t *, const cuuint32_t *, CUtensorMapInterleave,
                                    CUtensorMapSwizzle, CUtensorMapL2promotion, CUtensorMapFloatOOBfill);

static encode_tiled_fn step_encode_tiled() {
    static std::atomic<encode_tiled_fn> fn{nullptr};
    encode_tiled_fn f = fn.load(std::memory_order_acquire);
    if (!f) {
        void *p = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &p, cudaEnableDefault, &q) == cudaSuccess &&
            q == cudaDriverEntryPointSuccess)
            f = (encode_tiled_fn)p;
        else
            cudaGetLastError();
        fn.store(f, std::memory_order_release);
    }
    return f;
}

extern "C" size_t tm_cuda_program_bytes(uint32_t max_ops, uint64_t vector_elems, uint64_t attention_elems) {
    return max_ops ? program_bytes(max_ops, vector_elems + 4ull * max_ops, attention_elems) : 0;
}

extern "C" uint64_t tm_cuda_program_attention_elems(uint32_t heads, uint32_t head_dim, uint32_t cap) {
    return (uint64_t)heads * ((cap + kAttnSplit - 1) / kAttnSplit) * (head_dim + 2);
}

extern "C" int tm_cuda_program_supports_gemv(uint32_t cols) {
    return cols != 0 && cols % kChunkCols == 0 && cols <= kMaxQuads * kCThreads * 4;
}

extern "C" int tm_cuda_program_supports_attention(uint32_t heads, uint32_t kv_heads, uint32_t head_dim, uint32_t n_rot) {
    if (heads == 0 || kv_heads == 0 || heads % kv_heads != 0) return 0;
    const uint32_t g = heads / kv_heads;
    return (head_dim == 128 || head_dim == 256) && n_rot == head_dim && (g == 1 || g == 2 || g == 4);
}

static int program_push(tm_cuda_ctx *ctx, const step_op &op, uint32_t out_len, char *err, size_t err_cap) {
    tm_step_program *p = (tm_step_program *)ctx->program;
    if (p->ops.size() >= p->max_ops)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "the program was opened for %u operators", p->max_ops);
    p->ops.push_back(op);
    p->out_len.push_back(out_len);
    return TM_CUDA_OK;
}

int tm_step_record_gemv(tm_cuda_ctx *ctx, const void *q, const void *d, const float *x, float *y, const float *pro,
                        uint32_t rows, uint32_t cols, int prologue, int epilogue, float eps, uint32_t batch, char *err,
                        size_t err_cap) {
    tm_step_program *p = (tm_step_program *)ctx->program;
    if (batch != 1 || !tm_cuda_program_supports_gemv(cols))
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "a persistent program takes one-token GEMVs whose columns are a multiple of 64, at most %u "
                       "(got batch %u, %u columns)", kMaxQuads * kCThreads * 4, batch, cols);
    if (prologue == TM_CUDA_PRO_RMSNORM && cols > kNormQuads * kCThreads * 4)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "a persistent program norms GEMV inputs of at most %u columns (got %u)", kNormQuads * kCThreads * 4, cols);
    if ((((size_t)x | (size_t)pro | (size_t)y) & 15u) != 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "program GEMV operands must be 16-byte aligned");
    step_op op = {};
    op.kind = STEP_GEMV;
    op.first_cta = p->next_cta;
    op.rows = rows;
    op.cols = cols;
    op.prologue = (uint32_t)prologue;
    op.epilogue = (uint32_t)epilogue;
    op.eps = eps;
    op.p[0] = q; op.p[1] = d; op.p[2] = x; op.p[3] = y; op.p[4] = pro;
    const uint32_t units = (rows + 15u) / 16u;
    p->next_cta = (p->next_cta + units) % (uint32_t)ctx->sm_count;
    return program_push(ctx, op, rows, err, err_cap);
}

int tm_step_record_embed(tm_cuda_ctx *ctx, const void *q, const void *d, uint32_t rows, uint32_t cols,
                         const uint32_t *ids, uint32_t slot, const uint32_t *pos, int bias, uint32_t ids_len,
                         float scale, float *out, char *err, size_t err_cap) {
    step_op op = {};
    op.kind = STEP_EMBED;
    op.rows = rows;
    op.cols = cols;
    op.scale = scale;
    op.p[0] = q; op.p[1] = d; op.p[2] = ids; op.p[3] = pos; op.p[4] = out;
    op.u[0] = slot; op.u[1] = (uint32_t)bias; op.u[2] = ids_len;
    return program_push(ctx, op, cols, err, err_cap);
}

int tm_step_record_attention(tm_cuda_ctx *ctx, const float *q, const float *k, const float *v, const float *qn,
                             const float *kn, const float *inv_freq, void *kc, void *vc, float *out, float *scratch,
                             const uint32_t *pos, uint32_t *status, uint32_t heads, uint32_t kv_heads, uint32_t hd,
                             uint32_t n_rot, uint32_t cap, uint32_t window, float eps, float scale, int exact,
                             char *err, size_t err_cap) {
    tm_step_program *p = (tm_step_program *)ctx->program;
    (void)scratch;  // the program keeps the splits' partial results in its own flagged region
    if (exact || !tm_cuda_program_supports_attention(heads, kv_heads, hd, n_rot))
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "a persistent program takes the tolerance-qualified decode attention only: head dim 128 or "
                       "256 fully rotated, 1, 2 or 4 query heads per KV head (got %u/%u heads of %u, %u rotated, "
                       "exact %d)", heads, kv_heads, hd, n_rot, exact);
    if (tm_cuda_program_attention_elems(heads, hd, cap) > p->attn_words)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "attention of %u heads x %u at capacity %u needs %llu partial words; the program was opened "
                       "for %llu", heads, hd, cap, (unsigned long long)tm_cuda_program_attention_elems(heads, hd, cap),
                       (unsigned long long)p->attn_words);
    step_op op = {};
    op.kind = STEP_ATTN;
    op.eps = eps;
    op.scale = scale;
    op.p[0] = q; op.p[1] = k; op.p[2] = v; op.p[3] = qn; op.p[4] = kn; op.p[5] = inv_freq;
    op.p[6] = kc; op.p[7] = vc; op.p[8] = out; op.p[10] = pos; op.p[11] = status;
    op.u[0] = heads; op.u[1] = kv_heads; op.u[2] = hd; op.u[3] = cap; op.u[4] = window;
    return program_push(ctx, op, heads * hd, err, err_cap);
}

int tm_step_record_argmax(tm_cuda_ctx *ctx, const float *x, uint32_t n, uint32_t *out, uint32_t base,
                          const uint32_t *pos, uint32_t out_cap, uint32_t *mirror, char *err, size_t err_cap) {
    step_op op = {};
    op.kind = STEP_ARGMAX;
    op.p[0] = x; op.p[1] = out; op.p[2] = pos; op.p[3] = mirror;
    op.u[0] = n; op.u[1] = base; op.u[2] = out_cap;
    return program_push(ctx, op, 0, err, err_cap);
}

int tm_step_record_norm_add(tm_cuda_ctx *ctx, const float *pp, const float *w, float *x, uint32_t rows, uint32_t cols,
                            float eps, char *err, size_t err_cap) {
    if (rows != 1)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "a persistent program norms one row (got %u)", rows);
    step_op op = {};
    op.kind = STEP_NORM_ADD;
    op.cols = cols;
    op.eps = eps;
    op.p[0] = pp; op.p[1] = w; op.p[2] = x;
    return program_push(ctx, op, cols, err, err_cap);
}

int tm_step_record_pos_add(tm_cuda_ctx *ctx, uint32_t *counter, uint32_t delta, char *err, size_t err_cap) {
    tm_step_program *p = (tm_step_program *)ctx->program;
    step_op op = {};
    op.kind = STEP_POS_ADD;
    op.p[0] = counter;
    op.u[0] = delta;
    op.u[1] = p->pos_adds++;  // which of the program's position updates this is
    return program_push(ctx, op, 0, err, err_cap);
}

void tm_step_free(tm_cuda_ctx *ctx, tm_step_program *p) {
    if (!p) return;
    if (p->dev) {
        cudaFree(p->dev);
        ctx->allocated.fetch_sub(p->dev_bytes);
    }
    if (p->trace) cudaFree(p->trace);
    delete p;
}

int tm_step_launch(tm_cuda_ctx *ctx, tm_step_program *p, char *err, size_t err_cap) {
    step_params P = {};
    const uint32_t n_ops = (uint32_t)p->ops.size();
    P.ops = (const step_op *)p->dev;
    P.n_ops = n_ops;
    P.arrivals = (uint32_t *)(p->dev + p->ops_bytes);
    P.status = P.arrivals + 1;
    P.argmax_ll = (u64 *)(p->dev + p->ops_bytes + 256);
    P.attn_ll = (u64 *)(p->dev + p->attn_off);
    // sequence numbers: operator i of launch L carries 1 + (L * n_ops + i) mod (2^32 - 1 - n_ops): never 0
    // (the value of untouched memory), and a launch's range never meets its predecessor's
    const uint64_t span = 0xFFFFFFFFull - n_ops;
    P.seq_base = (uint32_t)((p->launches * n_ops) % span) + 1u;
    P.seq_skew = p->seq_skew;
    P.arrivals_base = (uint32_t)(p->launches * p->pos_adds * (uint64_t)p->grid);
    P.n_slots = p->n_slots;
    P.xs_bytes = p->xs_bytes;
    P.spin_limit = p->spin_limit;
    P.l2_ahead = p->l2_ahead;
    P.trace = p->trace;
    p->launches += 1;
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = dim3(p->grid);
    cfg.blockDim = dim3(kStepThreads);
    cfg.dynamicSmemBytes = p->smem;
    cfg.stream = ctx->stream;
    cudaLaunchAttribute at[1];
    at[0].id = cudaLaunchAttributeCooperative;  // every CTA resident at once: consumers poll what other CTAs produce
    at[0].val.cooperative = 1;
    cfg.attrs = at;
    cfg.numAttrs = 1;
    TM_CUDA_TRY(cudaLaunchKernelEx(&cfg, decode_step_kernel, P));
    return TM_CUDA_OK;
}

extern "C" {

int tm_cuda_begin_program(tm_cuda_ctx *ctx, uint32_t max_ops, uint64_t vector_elems, uint64_t attention_elems,
                          char *err, size_t err_cap) {
    TM_ENTER();
    if (ctx->group_open || ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "a dispatch group or program is already open");
    if (max_ops == 0 || max_ops > 65536)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "a program holds 1..65536 operators (asked for %u)", max_ops);
    if (ctx->sm_count > 1024)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "more than 1024 SMs");
    tm_step_program *p = new tm_step_program();
    p->max_ops = max_ops;
    p->ll_words = vector_elems + 4ull * max_ops;  // each vector starts on a 32-byte boundary
    p->attn_words = attention_elems;
    p->grid = ctx->sm_count;
    ctx->program = p;
    return TM_CUDA_OK;
}

int tm_cuda_abort_program(tm_cuda_ctx *ctx, char *err, size_t err_cap) {
    TM_ENTER();
    if (!ctx->program) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "no program is open");
    tm_step_free(ctx, (tm_step_program *)ctx->program);
    ctx->program = nullptr;
    return TM_CUDA_OK;
}

int tm_cuda_end_program(tm_cuda_ctx *ctx, tm_cuda_graph **out, char *err, size_t err_cap) {
    TM_ENTER();
    if (!out) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "null program output");
    tm_step_program *p = (tm_step_program *)ctx->program;
    if (!p) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "no program is open");
    ctx->program = nullptr;
    auto fail = [&](int code, const char *msg) {
        tm_step_free(ctx, p);
        return tm_fail(err, err_cap, code, "%s", msg);
    };
    if (p->ops.empty()) return fail(TM_CUDA_ERR_BOUNDS, "the program is empty");
    const size_t n = p->ops.size();
    // shared memory: the activation stage (or the attention groups), then as many ring stages as fit
    uint32_t xs = (kCThreads / 128) * kAttnSub;
    for (const step_op &op : p->ops)
        if (op.kind == STEP_GEMV) xs = std::max(xs, stage_bytes_for(op.cols));
    xs = (uint32_t)tm_round_up(xs, 128);
    const size_t budget = ctx->smem_optin;
    if ((size_t)xs + kTailBytes + 3u * kSlotBytes > budget)
        return fail(TM_CUDA_ERR_UNSUPPORTED, "the widest GEMV of the program leaves no room for the weight ring");
    uint32_t slots = (uint32_t)((budget - xs - kTailBytes) / kSlotBytes);
    if (slots > kMaxSlots) slots = kMaxSlots;
    if (const char *e = getenv("TM_CUDA_STEP_SLOTS")) {
        const uint32_t want = (uint32_t)strtoul(e, nullptr, 10);
        if (want >= 3 && want < slots) slots = want;
    }
    p->xs_bytes = xs;
    p->n_slots = slots;
    p->smem = xs + slots * kSlotBytes + kTailBytes;
    if (const char *e = getenv("TM_CUDA_STEP_SPIN")) p->spin_limit = (uint32_t)strtoul(e, nullptr, 10);
    if (const char *e = getenv("TM_CUDA_STEP_L2_AHEAD")) p->l2_ahead = (uint32_t)strtoul(e, nullptr, 10);
    // device memory: operator table | arrivals, status | argmax words | tensor maps | flagged vectors | attention partials
    p->ops_bytes = tm_round_up((size_t)p->max_ops * sizeof(step_op), 256);
    p->maps_off = p->ops_bytes + 256 + 2 * 8 * 1024;
    p->ll_off = p->maps_off + (size_t)p->max_ops * 128;
    p->attn_off = p->ll_off + tm_round_up((size_t)p->ll_words * 8, 256);
    p->dev_bytes = program_bytes(p->max_ops, p->ll_words, p->attn_words);
    // flagged regions and sources: every operator's output gets its own region (written once per launch);
    // an input that an earlier operator of the program produces is read from that operator's region
    std::vector<uint64_t> region(n, 0);
    uint64_t used = 0;
    for (size_t i = 0; i < n; ++i) {
        region[i] = used;
        used += (p->out_len[i] + 3u) / 4u * 4u;
    }
    if (used > p->ll_words) return fail(TM_CUDA_ERR_BOUNDS, "the program's vectors exceed the elements it was opened for");
    auto out_ptr = [&](size_t j) -> const float * {
        const step_op &o = p->ops[j];
        switch (o.kind) {
            case STEP_GEMV: return (const float *)o.p[3];
            case STEP_EMBED: return (const float *)o.p[4];
            case STEP_ATTN: return (const float *)o.p[8];
            case STEP_NORM_ADD: return (const float *)o.p[2];
            default: return nullptr;
        }
    };
    bool bad_overlap = false;
    // source of `len` floats at `ptr` for operator i: the latest earlier operator whose output holds them all
    auto resolve = [&](size_t i, const float *ptr, uint32_t len, int slot) {
        step_op &op = p->ops[i];
        op.in[slot] = nullptr;
        op.in_op[slot] = 0;
        if (!ptr || len == 0) return;
        for (size_t j = i; j-- > 0;) {
            const float *o = out_ptr(j);
            if (!o || p->out_len[j] == 0) continue;
            const float *oe = o + p->out_len[j], *pe = ptr + len;
            if (pe <= o || ptr >= oe) continue;          // disjoint
            if (ptr < o || pe > oe) { bad_overlap = true; return; }  // straddles an output
            op.in[slot] = (const u64 *)nullptr + (region[j] + (uint64_t)(ptr - o));  // element offset, rebased below
            op.in_op[slot] = (uint32_t)j;
            op.pad[slot] = 1;  // marks "resolved" until the rebase
            return;
        }
    };
    for (size_t i = 0; i < n; ++i) {
        step_op &op = p->ops[i];
        op.pad[0] = op.pad[1] = op.pad[2] = 0;
        switch (op.kind) {
            case STEP_GEMV:
                resolve(i, (const float *)op.p[2], op.cols, 0);
                if (op.prologue == TM_CUDA_PRO_SILU_MUL || op.prologue == TM_CUDA_PRO_GELU_MUL)
                    resolve(i, (const float *)op.p[4], op.cols, 1);
                if (op.epilogue == TM_CUDA_EPI_ADD) resolve(i, (const float *)op.p[3], op.rows, 2);
                break;
            case STEP_ATTN:
                resolve(i, (const float *)op.p[0], op.u[0] * op.u[2], 0);
                resolve(i, (const float *)op.p[1], op.u[1] * op.u[2], 1);
                resolve(i, (const float *)op.p[2], op.u[1] * op.u[2], 2);
                break;
            case STEP_ARGMAX: resolve(i, (const float *)op.p[0], op.u[0], 0); break;
            case STEP_NORM_ADD:
                resolve(i, (const float *)op.p[0], op.cols, 0);
                resolve(i, (const float *)op.p[2], op.cols, 1);
                break;
            default: break;
        }
    }
    if (bad_overlap) return fail(TM_CUDA_ERR_UNSUPPORTED, "an operator reads a range that straddles another operator's output");
    void *table = nullptr;
    if (cudaMalloc(&table, p->dev_bytes) != cudaSuccess) {
        cudaGetLastError();
        return fail(TM_CUDA_ERR_ALLOC, "allocating the program failed");
    }
    p->dev = (unsigned char *)table;
    ctx->allocated.fetch_add(p->dev_bytes);
    // one tensor map per GEMV: the int8 plane as [rows][cols / 4] 32-bit words (a box side is at most 256
    // elements: 256 words = the 1024 bytes of a stage row), box = 16 rows x min(1024, cols) bytes, no swizzle
    std::vector<CUtensorMap> maps(n);
    {
        encode_tiled_fn encode = step_encode_tiled();
        if (!encode) {
            tm_step_free(ctx, p);
            return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "the driver does not export cuTensorMapEncodeTiled");
        }
        for (size_t i = 0; i < n; ++i) {
            step_op &op = p->ops[i];
            if (op.kind != STEP_GEMV) continue;
            op.row_stride = op.cols < kStageCols ? op.cols : kStageCols;
            const cuuint64_t gdim[2] = {op.cols / 4u, op.rows};
            const cuuint64_t gstride[1] = {(cuuint64_t)op.cols};
            const cuuint32_t box[2] = {op.row_stride / 4u, 16u};
            const cuuint32_t estr[2] = {1, 1};
            const CUresult cr = encode(&maps[i], CU_TENSOR_MAP_DATA_TYPE_UINT32, 2, (void *)op.p[0], gdim, gstride, box, estr,
                                       CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_NONE,
                                       CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
            if (cr != CUDA_SUCCESS) {
                tm_step_free(ctx, p);
                return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "cuTensorMapEncodeTiled failed (%d) for a %u x %u matrix",
                               (int)cr, op.rows, op.cols);
            }
            op.wmap = p->dev + p->maps_off + i * 128;
        }
    }
    u64 *ll = (u64 *)(p->dev + p->ll_off);
    for (size_t i = 0; i < n; ++i) {
        step_op &op = p->ops[i];
        op.out = p->out_len[i] ? ll + region[i] : nullptr;
        for (int s = 0; s < 3; ++s) {
            if (op.pad[s]) {
                op.in[s] = ll + (size_t)(op.in[s] - (const u64 *)nullptr);
                if ((size_t)op.in[s] % 32 != 0 && op.kind == STEP_GEMV && s < 2) {
                    tm_step_free(ctx, p);
                    return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                                   "a GEMV input starts %zu floats into another operator's output: not a multiple of 4",
                                   (size_t)((op.in[s] - ll) - region[op.in_op[s]]));
                }
            }
            op.pad[s] = 0;
        }
        // the plain vector is stored by the LAST operator that writes the buffer
        op.write_plain = 1;
        const float *mine = out_ptr(i);
        for (size_t j = i + 1; j < n && mine; ++j) {
            const float *o = out_ptr(j);
            if (o && o < mine + p->out_len[i] && mine < o + p->out_len[j]) {
                op.write_plain = 0;
                break;
            }
        }
    }
    static std::atomic<bool> attr_done[64] = {};
    const int dev = ctx->device;
    if (dev < 0 || dev >= 64 || !attr_done[dev].load(std::memory_order_acquire)) {
        if (cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)budget) != cudaSuccess) {
            cudaGetLastError();
            return fail(TM_CUDA_ERR_INTERNAL, "cannot raise the persistent kernel's shared memory limit");
        }
        if (dev >= 0 && dev < 64) attr_done[dev].store(true, std::memory_order_release);
    }
    // shared memory the kernel does not ask for stays L1 (local memory of a register-hungry thread lives there)
    cudaFuncSetAttribute(decode_step_kernel, cudaFuncAttributePreferredSharedMemoryCarveout,
                         (int)((p->smem + 1024) * 100 / (228 * 1024) + 1));
    cudaGetLastError();
    int per_sm = 0;
    if (cudaOccupancyMaxActiveBlocksPerMultiprocessor(&per_sm, decode_step_kernel, kStepThreads, p->smem) != cudaSuccess ||
        per_sm < 1) {
        cudaGetLastError();
        return fail(TM_CUDA_ERR_INTERNAL, "the persistent kernel does not fit an SM");
    }
    if (cudaMemsetAsync(p->dev, 0, p->dev_bytes, ctx->stream) != cudaSuccess ||
        cudaMemcpyAsync(p->dev, p->ops.data(), n * sizeof(step_op), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess ||
        cudaMemcpyAsync(p->dev + p->maps_off, maps.data(), n * sizeof(CUtensorMap), cudaMemcpyHostToDevice, ctx->stream) != cudaSuccess ||
        cudaStreamSynchronize(ctx->stream) != cudaSuccess) {
        cudaGetLastError();
        return fail(TM_CUDA_ERR_INTERNAL, "uploading the program failed");
    }
    tm_cuda_graph *g = new tm_cuda_graph();
    g->owner = ctx;
    g->program = p;
    g->kernels = 1;
    ctx->graphs.insert(g);
    *out = g;
    return TM_CUDA_OK;
}

int tm_cuda_program_status(tm_cuda_ctx *ctx, tm_cuda_graph *graph, uint32_t *status, char *err, size_t err_cap) {
    TM_ENTER();
    if (!graph || ctx->graphs.find(graph) == ctx->graphs.end() || !graph->program || !status)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "not a program of this context");
    tm_step_program *p = (tm_step_program *)graph->program;
    TM_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    TM_CUDA_TRY(cudaMemcpy(status, p->dev + p->ops_bytes + 4, 4, cudaMemcpyDeviceToHost));
    return TM_CUDA_OK;
}

// Per-operator time stamps of CTA 0 in the program's LAST launch (nanoseconds of the device's global
// timer): out[8*i + 0] = operator i started, [1] = its activations were staged (GEMV), [2] = its work
// on this CTA was done, [7] = the weight producer reached it.  The first call switches tracing on (and
// returns zeros); a profiling aid.
int tm_cuda_program_trace(tm_cuda_ctx *ctx, tm_cuda_graph *graph, uint64_t *out, uint32_t max_ops, uint32_t *kinds,
                          char *err, size_t err_cap) {
    TM_ENTER();
    if (!graph || ctx->graphs.find(graph) == ctx->graphs.end() || !graph->program || !out)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "not a program of this context");
    tm_step_program *p = (tm_step_program *)graph->program;
    const size_t n = p->ops.size();
    if (max_ops < n) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "the program has %zu operators", n);
    TM_CUDA_TRY(cudaStreamSynchronize(ctx->stream));
    if (!p->trace) {
        TM_CUDA_TRY(cudaMalloc((void **)&p->trace, n * 8 * 8));
        TM_CUDA_TRY(cudaMemset(p->trace, 0, n * 8 * 8));
    }
    TM_CUDA_TRY(cudaMemcpy(out, p->trace, n * 8 * 8, cudaMemcpyDeviceToHost));
    if (kinds)
        for (size_t i = 0; i < n; ++i) kinds[i] = p->ops[i].kind;
    return TM_CUDA_OK;
}

int tm_cuda_program_debug(tm_cuda_ctx *ctx, tm_cuda_graph *graph, uint32_t sequence_skew, uint32_t spin_limit,
                          char *err, size_t err_cap) {
    TM_ENTER();
    if (!graph || ctx->graphs.find(graph) == ctx->graphs.end() || !graph->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "not a program of this context");
    tm_step_program *p = (tm_step_program *)graph->program;
    p->seq_skew = sequence_skew;
    if (spin_limit) p->spin_limit = spin_limit;
    return TM_CUDA_OK;
}

}  // extern "C"
