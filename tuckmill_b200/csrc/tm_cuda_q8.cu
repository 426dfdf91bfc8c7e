// Q8_0 weights: plane repacking, the decode GEMV / exact batched GEMM, and the
// embedding-row dequantisers.
//
// Arithmetic contract (the reference's device GEMV, native/metal/kernels.metal:
// 72-118, and its batched twin :434-476): y[r] = sum over blocks of
// d_{r,b} * sum_l q_{r,b,l} * x[32b+l] with f32 accumulation, reduction order
// free (tolerance-registered against the scalar CPU order,
// crates/tuckcore/src/kernels.rs:186-204).  The design is not the Metal
// kernel's; it is described at q8_gemv_kernel below.
#include <type_traits>

#include "tm_cuda_internal.cuh"
#include "tm_cuda_device.cuh"

namespace {

constexpr int kThreads = tmdev::kThreads;  // 8 warps per CTA
constexpr int kWarps = tmdev::kWarps;
using tmdev::block_sumsq;
using tmdev::silu_f;
using tmdev::gelu_tanh_f;
constexpr int kChunkCols = 64;  // columns one m16n8k32 pair covers (two Q8_0 blocks)

__device__ __forceinline__ int4 ldg_stream(const int4 *p) {
    int4 v;
    asm("ld.global.nc.L1::no_allocate.v4.s32 {%0,%1,%2,%3}, [%4];"
                 : "=r"(v.x), "=r"(v.y), "=r"(v.z), "=r"(v.w)
                 : "l"(p));
    return v;
}

// D += A(16x32 s8, row) * B(32x8 s8, col), s32 accumulate.
__device__ __forceinline__ void mma_s8(int (&d)[4], int a0, int a1, int a2, int a3, int b0, int b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k32.row.col.s32.s8.s8.s32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, "
        "{%0,%1,%2,%3};"
        : "+r"(d[0]), "+r"(d[1]), "+r"(d[2]), "+r"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}

struct gemv_args {
    const signed char *q;   // [rows][cols]
    const __half *d;        // [rows][cols/32]
    const float *x;         // [M][cols] (token stride = cols)
    float *y;               // [M][rows] (token stride = rows)
    const float *pro;       // norm weight [cols] or the `up` operand [M][cols]
    uint32_t rows, cols;
    uint32_t y_stride;      // floats between the outputs of consecutive tokens (the whole matrix's rows)
    float eps;
    int prologue, epilogue;
    uint32_t plane;         // bytes between digit planes (== 64 mod 128)
    uint32_t ks;            // column splits per row tile (1, 2, 4 or 8)
    uint32_t shape_rows;    // host only: rows of the matrix the column split is chosen for (a row view: its parent's)
    // kAdd forms only: x' = x + rmsnorm(add_p, add_w, eps) is formed first (a layer's output norm and
    // residual add, folded into the projection that consumes the result), multiplied after the prologue's
    // own norm, and written to x_out by CTA 0 (a buffer other than x: every CTA reads x).
    const float *add_p = nullptr, *add_w = nullptr;
    float *x_out = nullptr;
};

// Bytes of shared memory one token's staged activations take.
__host__ __device__ inline size_t token_smem(uint32_t cols, uint32_t plane) {
    return 4u * (size_t)plane + (size_t)(cols / 32u) * 16u;
}

/*
 * The decode GEMV, HBM-bound by construction: the int8 quants go from global
 * memory straight into the A operand of the integer tensor-core MMA, with no
 * per-weight conversion at all.  To keep f32 accuracy the f32 activations are
 * split, once per CTA, into four signed 7-bit digits against a power-of-two
 * block scale: x = 2^e * (a0 + a1/2^7 + a2/2^14 + a3/2^21), exact for every
 * element whose bits lie within 2^-27 of its block's largest magnitude.  The
 * digits of the two blocks of a 64-column chunk are the eight B columns, so
 * one accumulator tile holds sum(q * a_k) per (row, block, digit) exactly in
 * s32; f32 work is 4 conversions and 6 FMAs per 32 weights:
 *     y[r] += d[r,b] * sum_k float(S[r,b,k]) * 2^(e_b - 7k).
 * A warp owns a 16-row tile; lane (g, t) loads 16 quants of rows g and g+8 at
 * columns chunk*64 + t*16.  `ks` warps split the chunks of a tile (interleaved)
 * and their partial row sums are added in a fixed order, so small matrices
 * still spread over the machine.  ks and the lane mapping depend only on the
 * matrix shape, never on the batch, which keeps a (row, token) result
 * bit-identical between the GEMV and any batched call.
 */
template <int M, int kSlots, int H, bool kAdd = false>
__global__ void __launch_bounds__(kThreads) q8_gemv_kernel(const gemv_args a) {
    extern __shared__ __align__(16) unsigned char smem[];
    __shared__ float red[kWarps];
    __shared__ float partial[kWarps][M][16];
    const uint32_t cols = a.cols, rows = a.rows, nb = cols / 32u, plane = a.plane;
    const size_t tok = token_smem(cols, plane);
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5;
    const int g = lane >> 2, t4 = lane & 3;

    const uint32_t ks = a.ks, tiles_per_cta = kWarps / ks;
    const uint32_t my_ks = warp % ks, my_tile = warp / ks;
    const uint32_t n_tiles = (rows + 15u) / 16u;
    const uint32_t n_chunks = (cols + kChunkCols - 1u) / kChunkCols;

    // Weights do not depend on the activations, so they stream through registers on their own
    // schedule: the warp's (tile, chunk) work is one flat sequence of groups of H chunks, held in
    // kSlots register slots.  While one slot is multiplied the other slots' loads are in flight, and
    // a slot is refilled (with the group kSlots ahead, possibly of the warp's NEXT tile) as soon as it
    // has been consumed -- loads never stop at a tile boundary.  The first kSlots groups are
    // requested before the activations are staged, so both latencies overlap.
    // kSlots x H is chosen per shape by the host: three slots of two chunks keep the short column
    // ranges of the small projections streaming; one slot of six (a load / multiply alternation with
    // wide bursts per row: the most bytes in flight the register file allows at two CTAs per SM) is the
    // register form for long ranges.
    // kSlots == 0 selects the third form, used for the tall matrices: the stream goes through a
    // per-warp ring of H chunk slots in SHARED memory filled with cp.async (every lane copies, and
    // later reads back, its own 16 bytes of rows g and g+8; the chunk's scale pairs ride along as
    // 4-byte copies).  Bytes in flight then cost no registers: H = 8..12 chunks per warp.
    constexpr bool kAsync = kSlots == 0;
    constexpr int U = kAsync ? 1 : kSlots * H;  // chunks in registers
    constexpr uint32_t kRingSlot = 1024u + 64u;  // 2 x 512 bytes of quants + 16 rows x 2 scales
    int4 wa[U], wb[U];
    unsigned short ha[U], hb[U];
    const uint32_t tile_stride = gridDim.x * tiles_per_cta;
    uint32_t ld_tile = blockIdx.x * tiles_per_cta + my_tile, ld_ch = my_ks;  // next group to request
    auto load_half = [&](auto half_c) {
        constexpr int half = decltype(half_c)::value;
        if (ld_tile >= n_tiles) return;
        const uint32_t row_a = min(ld_tile * 16u + g, rows - 1u), row_b = min(ld_tile * 16u + g + 8u, rows - 1u);
        const signed char *pa = a.q + (size_t)row_a * cols + t4 * 16u;
        const signed char *pb = a.q + (size_t)row_b * cols + t4 * 16u;
        const unsigned short *sa = (const unsigned short *)a.d + (size_t)row_a * nb + (t4 >> 1);
        const unsigned short *sb = (const unsigned short *)a.d + (size_t)row_b * nb + (t4 >> 1);
#pragma unroll
        for (int u = 0; u < H; ++u) {
            const uint32_t ch = ld_ch + u * ks;
            const bool inb = ch < n_chunks && ch * kChunkCols + t4 * 16u < cols;
            wa[half * H + u] = wb[half * H + u] = make_int4(0, 0, 0, 0);
            ha[half * H + u] = hb[half * H + u] = 0;
            if (inb) {
                wa[half * H + u] = ldg_stream((const int4 *)(pa + (size_t)ch * kChunkCols));
                wb[half * H + u] = ldg_stream((const int4 *)(pb + (size_t)ch * kChunkCols));
                ha[half * H + u] = __ldg(sa + ch * 2u);
                hb[half * H + u] = __ldg(sb + ch * 2u);
            }
        }
        ld_ch += H * ks;
        if (ld_ch >= n_chunks) {
            ld_ch = my_ks;
            ld_tile += tile_stride;
        }
    };
    using half0 = std::integral_constant<int, 0>;
    using half1 = std::integral_constant<int, 1>;
    using half2 = std::integral_constant<int, 2>;
    const uint32_t ring = (uint32_t)__cvta_generic_to_shared(smem) + (uint32_t)(((size_t)M * tok + 15u) & ~(size_t)15u) +
                          (uint32_t)warp * (uint32_t)(H > 0 ? H : 1) * kRingSlot;
    // One chunk of the flat sequence into ring slot `slot` (always commits a group, so exactly H
    // groups are outstanding at any time and wait_group H-1 means "the oldest has landed").
    auto async_issue = [&](uint32_t slot) {
        if (ld_tile < n_tiles) {
            const uint32_t row_a = min(ld_tile * 16u + g, rows - 1u), row_b = min(ld_tile * 16u + g + 8u, rows - 1u);
            const uint32_t dst = ring + slot * kRingSlot;
            const size_t col = (size_t)ld_ch * kChunkCols + t4 * 16u;
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + (uint32_t)lane * 16u),
                         "l"(a.q + (size_t)row_a * cols + col) : "memory");
            asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst + 512u + (uint32_t)lane * 16u),
                         "l"(a.q + (size_t)row_b * cols + col) : "memory");
            if (t4 < 2) {  // the two block scales of this chunk for row g (t4 = 0) / g + 8 (t4 = 1)
                const uint32_t r16 = (uint32_t)g + 8u * (uint32_t)t4;
                const unsigned short *sp = (const unsigned short *)a.d + (size_t)(t4 == 0 ? row_a : row_b) * nb + ld_ch * 2u;
                asm volatile("cp.async.ca.shared.global [%0], [%1], 4;" ::"r"(dst + 1024u + r16 * 4u), "l"(sp) : "memory");
            }
            ld_ch += ks;
            if (ld_ch >= n_chunks) {
                ld_ch = my_ks;
                ld_tile += tile_stride;
            }
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    if constexpr (kAsync) {
#pragma unroll
        for (int i = 0; i < H; ++i) async_issue((uint32_t)i);
    } else {
        load_half(half0{});
        if constexpr (kSlots > 1) load_half(half1{});
        if constexpr (kSlots > 2) load_half(half2{});
    }
    if (ld_tile < n_tiles) {  // the groups after those: towards L2
        const uint32_t row_a = min(ld_tile * 16u + g, rows - 1u), row_b = min(ld_tile * 16u + g + 8u, rows - 1u);
#pragma unroll
        for (uint32_t j = 0; j < 4; ++j) {
            const uint32_t c0 = (ld_ch + j * ks) * kChunkCols + t4 * 16u;
            if (c0 < cols) {
                asm volatile("prefetch.global.L2 [%0];" ::"l"(a.q + (size_t)row_a * cols + c0));
                asm volatile("prefetch.global.L2 [%0];" ::"l"(a.q + (size_t)row_b * cols + c0));
            }
        }
    }

    tmdev::pdl_trigger();
    tmdev::pdl_wait();  // the activations (and y, for the accumulate epilogue) come from the predecessor

    // ---- stage the activations: elementwise prologue, then digit planes ----
#pragma unroll 1
    for (int m = 0; m < M; ++m) {
        const float *xm = a.x + (size_t)m * cols;
        signed char *dig = (signed char *)(smem + (size_t)m * tok);
        float *coef = (float *)(smem + (size_t)m * tok + 4u * (size_t)plane);
        // Each thread takes 4 consecutive columns, so 8 adjacent lanes own one
        // 32-column block; kBatch such quads are loaded before any is digitised.
        constexpr int kBatch = 4;
        // Up to 4096 columns the whole row sits in one batch of registers and the
        // RMS norm's sum of squares is taken from them (one trip to memory);
        // wider rows make a separate pass first.  Same canonical tree either way.
        const bool one_pass = cols <= (uint32_t)(kThreads * 4 * kBatch);
        float inv_rms = 0.0f;
        if (a.prologue == TM_CUDA_PRO_RMSNORM && !one_pass) {
            const float ss = block_sumsq(xm, cols, red);
            inv_rms = 1.0f / sqrtf(ss / (float)cols + a.eps);
        }
        const bool vec_ok = (((size_t)xm | (size_t)a.pro) & 15u) == 0 && (cols & 3u) == 0;
#pragma unroll 1
        for (uint32_t cb = 0; cb < cols; cb += kThreads * 4 * kBatch) {
            float4 vs[kBatch], ps[kBatch];
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                const uint32_t c = cb + (i * kThreads + threadIdx.x) * 4u;
                vs[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                ps[i] = make_float4(1.f, 1.f, 1.f, 1.f);
                if (c < cols) {
                    const float *pp = a.prologue == TM_CUDA_PRO_RMSNORM ? a.pro + c
                                      : a.prologue != TM_CUDA_PRO_NONE ? a.pro + (size_t)m * cols + c
                                                                       : nullptr;
                    if (vec_ok) {
                        vs[i] = *(const float4 *)(xm + c);
                        if (pp) ps[i] = *(const float4 *)pp;
                    } else {
                        vs[i] = make_float4(xm[c], xm[c + 1], xm[c + 2], xm[c + 3]);
                        if (pp) ps[i] = make_float4(pp[0], pp[1], pp[2], pp[3]);
                    }
                }
            }
            if constexpr (kAdd) {
                // x' = x + rmsnorm(p) * w, rounded like the stand-alone operator (two multiplies, one add);
                // the host selects this form only for one-pass widths with the norm prologue
                float4 pv[kBatch], aw[kBatch];
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    const uint32_t c = cb + (i * kThreads + threadIdx.x) * 4u;
                    pv[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    aw[i] = make_float4(0.f, 0.f, 0.f, 0.f);
                    if (c < cols) {
                        if (vec_ok && (((size_t)a.add_p | (size_t)a.add_w) & 15u) == 0) {
                            pv[i] = *(const float4 *)(a.add_p + c);
                            aw[i] = *(const float4 *)(a.add_w + c);
                        } else {
                            pv[i] = make_float4(a.add_p[c], a.add_p[c + 1], a.add_p[c + 2], a.add_p[c + 3]);
                            aw[i] = make_float4(a.add_w[c], a.add_w[c + 1], a.add_w[c + 2], a.add_w[c + 3]);
                        }
                    }
                }
                float sqp = 0.0f;
#pragma unroll
                for (int i = 0; i < kBatch; ++i) sqp = tmdev::sumsq_quad(sqp, pv[i]);
                const float inv_add = 1.0f / sqrtf(tmdev::block_reduce_sumsq(sqp, red) / (float)cols + a.eps);
#pragma unroll
                for (int i = 0; i < kBatch; ++i) {
                    vs[i].x = __fadd_rn(vs[i].x, __fmul_rn(__fmul_rn(pv[i].x, inv_add), aw[i].x));
                    vs[i].y = __fadd_rn(vs[i].y, __fmul_rn(__fmul_rn(pv[i].y, inv_add), aw[i].y));
                    vs[i].z = __fadd_rn(vs[i].z, __fmul_rn(__fmul_rn(pv[i].z, inv_add), aw[i].z));
                    vs[i].w = __fadd_rn(vs[i].w, __fmul_rn(__fmul_rn(pv[i].w, inv_add), aw[i].w));
                    const uint32_t c = cb + (i * kThreads + threadIdx.x) * 4u;
                    if (blockIdx.x == 0 && c < cols) {
                        if ((((size_t)a.x_out) & 15u) == 0 && (cols & 3u) == 0) *(float4 *)(a.x_out + c) = vs[i];
                        else { a.x_out[c] = vs[i].x; a.x_out[c + 1] = vs[i].y; a.x_out[c + 2] = vs[i].z; a.x_out[c + 3] = vs[i].w; }
                    }
                }
            }
            if (a.prologue == TM_CUDA_PRO_RMSNORM && one_pass) {
                float sq = 0.0f;  // thread t owns quads t, t+256, ... in this order (zero quads add nothing)
#pragma unroll
                for (int i = 0; i < kBatch; ++i) sq = tmdev::sumsq_quad(sq, vs[i]);
                inv_rms = 1.0f / sqrtf(tmdev::block_reduce_sumsq(sq, red) / (float)cols + a.eps);
            }
#pragma unroll
            for (int i = 0; i < kBatch; ++i) {
                const uint32_t c = cb + (i * kThreads + threadIdx.x) * 4u;
                // Whole warps leave together: 32 lanes x 4 columns = 128 columns, and
                // cols is a multiple of 32, so a partially filled warp keeps its
                // out-of-range lanes (zeros) in the shuffles below.
                if (cb + (i * kThreads + (threadIdx.x & ~31u)) * 4u >= cols) break;
                float v[4] = {vs[i].x, vs[i].y, vs[i].z, vs[i].w};
                const float pw[4] = {ps[i].x, ps[i].y, ps[i].z, ps[i].w};
                float amax = 0.0f;
#pragma unroll
                for (int j = 0; j < 4; ++j) {
                    if (a.prologue == TM_CUDA_PRO_RMSNORM) v[j] = v[j] * inv_rms * pw[j];
                    else if (a.prologue == TM_CUDA_PRO_SILU_MUL) v[j] = silu_f(v[j]) * pw[j];
                    else if (a.prologue == TM_CUDA_PRO_GELU_MUL) v[j] = gelu_tanh_f(v[j]) * pw[j];
                    // a non-finite value poisons its block (amax = inf -> NaN coefficient)
                    amax = fmaxf(amax, fabsf(v[j]) <= 3.402823466e38f ? fabsf(v[j]) : INFINITY);
                }
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 1));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 2));
                amax = fmaxf(amax, __shfl_xor_sync(0xffffffffu, amax, 4));
                if (c < cols) {
                    const bool bad = !(amax <= 3.402823466e38f);
                    int e = (int)((__float_as_uint(amax) >> 23) & 0xffu) - 127 - 5;
                    e = e < -100 ? -100 : e > 122 ? 122 : e;  // blocks below 2^-94 digitise to (near) zero
                    const float inv = __uint_as_float((uint32_t)(127 - e) << 23);
                    // t = v * 2^-e (|t| < 64, exact) is rounded once to a multiple of 2^-21
                    // and split into balanced base-128 digits with integer arithmetic:
                    // T = a0 2^21 + a1 2^14 + a2 2^7 + a3, a1..a3 in [-64, 63].
                    const float inv21 = inv * 2097152.0f;
                    uint32_t w0 = 0, w1 = 0, w2 = 0, w3 = 0;
#pragma unroll
                    for (int j = 0; j < 4; ++j) {
                        int T = __float2int_rn(v[j] * inv21);
                        const int a3 = (int)((uint32_t)T << 25) >> 25;
                        T = (T - a3) >> 7;
                        const int a2 = (int)((uint32_t)T << 25) >> 25;
                        T = (T - a2) >> 7;
                        const int a1 = (int)((uint32_t)T << 25) >> 25;
                        const int a0 = (T - a1) >> 7;
                        w0 |= ((uint32_t)a0 & 0xffu) << (8 * j);
                        w1 |= ((uint32_t)a1 & 0xffu) << (8 * j);
                        w2 |= ((uint32_t)a2 & 0xffu) << (8 * j);
                        w3 |= ((uint32_t)a3 & 0xffu) << (8 * j);
                    }
                    *(uint32_t *)(dig + c) = w0;
                    *(uint32_t *)(dig + plane + c) = w1;
                    *(uint32_t *)(dig + 2u * plane + c) = w2;
                    *(uint32_t *)(dig + 3u * plane + c) = w3;
                    const int k = lane & 7;
                    if (k < 4) {
                        const int ex = 127 + e - 7 * k;  // 2^(e - 7k); below the normal range -> 0
                        float sc = ex > 0 ? __uint_as_float((uint32_t)ex << 23) : 0.0f;
                        if (amax == 0.0f) sc = 0.0f;
                        if (bad) sc = __uint_as_float(0x7fc00000u);
                        coef[(c >> 5) * 4u + k] = sc;
                    }
                }
            }
        }
    }
    __syncthreads();

    const bool b_live = (t4 >> 1) == (g >> 2);  // this lane's k-slots belong to column n = g's block

    uint32_t cur_half = 0;  // the slot holding the next group to multiply
    auto multiply_half = [&](auto half_c, uint32_t ch0, float (&acc)[M][2]) {
        constexpr int half = decltype(half_c)::value;
#pragma unroll
        for (int u = 0; u < H; ++u) {
            const uint32_t ch = ch0 + u * ks;
            const uint32_t c0 = ch * kChunkCols + t4 * 16u;
            const bool inb = ch < n_chunks && c0 < cols;
            if (ch >= n_chunks) break;
            const float da = __half2float(__ushort_as_half(ha[half * H + u]));
            const float db = __half2float(__ushort_as_half(hb[half * H + u]));
            const int4 qa = wa[half * H + u], qb = wb[half * H + u];
#pragma unroll
            for (int m = 0; m < M; ++m) {
                const unsigned char *tokp = smem + (size_t)m * tok;
                int4 bx = make_int4(0, 0, 0, 0);
                if (b_live) bx = *(const int4 *)(tokp + (size_t)(g & 3) * plane + c0);
                int dd[4] = {0, 0, 0, 0};
                mma_s8(dd, qa.x, qb.x, qa.y, qb.y, bx.x, bx.y);
                mma_s8(dd, qa.z, qb.z, qa.w, qb.w, bx.z, bx.w);
                if (inb) {
                    const float2 cx = *(const float2 *)(tokp + 4u * (size_t)plane +
                                                        ((size_t)(c0 >> 5) * 4u + 2u * (t4 & 1)) * 4u);
                    const float va = fmaf((float)dd[1], cx.y, (float)dd[0] * cx.x);
                    const float vb = fmaf((float)dd[3], cx.y, (float)dd[2] * cx.x);
                    acc[m][0] = fmaf(da, va, acc[m][0]);
                    acc[m][1] = fmaf(db, vb, acc[m][1]);
                }
            }
        }
        load_half(half_c);  // refill with the group kSlots ahead
    };

    for (uint32_t base = blockIdx.x * tiles_per_cta; base < n_tiles; base += gridDim.x * tiles_per_cta) {
        const uint32_t tile = base + my_tile;
        const bool tile_ok = tile < n_tiles;
        float acc[M][2];
#pragma unroll
        for (int m = 0; m < M; ++m) acc[m][0] = acc[m][1] = 0.0f;

        if constexpr (kAsync) {
            if (tile_ok) {
#pragma unroll 1
                for (uint32_t ch = my_ks; ch < n_chunks; ch += ks) {
                    asm volatile("cp.async.wait_group %0;" ::"n"(H > 0 ? H - 1 : 0) : "memory");
                    __syncwarp();  // the scale pairs were copied by other lanes
                    const uint32_t src = ring + cur_half * kRingSlot;
                    int4 qa, qb;
                    unsigned short sa16, sb16;
                    asm volatile("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(qa.x), "=r"(qa.y), "=r"(qa.z), "=r"(qa.w) : "r"(src + (uint32_t)lane * 16u));
                    asm volatile("ld.shared.v4.s32 {%0,%1,%2,%3}, [%4];" : "=r"(qb.x), "=r"(qb.y), "=r"(qb.z), "=r"(qb.w) : "r"(src + 512u + (uint32_t)lane * 16u));
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sa16) : "r"(src + 1024u + (uint32_t)g * 4u + (uint32_t)(t4 >> 1) * 2u));
                    asm volatile("ld.shared.u16 %0, [%1];" : "=h"(sb16) : "r"(src + 1024u + (uint32_t)(g + 8) * 4u + (uint32_t)(t4 >> 1) * 2u));
                    const uint32_t c0 = ch * kChunkCols + t4 * 16u;
                    const float da = __half2float(__ushort_as_half(sa16));
                    const float db = __half2float(__ushort_as_half(sb16));
#pragma unroll
                    for (int m = 0; m < M; ++m) {
                        const unsigned char *tokp = smem + (size_t)m * tok;
                        int4 bx = make_int4(0, 0, 0, 0);
                        if (b_live) bx = *(const int4 *)(tokp + (size_t)(g & 3) * plane + c0);
                        int dd[4] = {0, 0, 0, 0};
                        mma_s8(dd, qa.x, qb.x, qa.y, qb.y, bx.x, bx.y);
                        mma_s8(dd, qa.z, qb.z, qa.w, qb.w, bx.z, bx.w);
                        const float2 cx = *(const float2 *)(tokp + 4u * (size_t)plane +
                                                            ((size_t)(c0 >> 5) * 4u + 2u * (t4 & 1)) * 4u);
                        const float va = fmaf((float)dd[1], cx.y, (float)dd[0] * cx.x);
                        const float vb = fmaf((float)dd[3], cx.y, (float)dd[2] * cx.x);
                        acc[m][0] = fmaf(da, va, acc[m][0]);
                        acc[m][1] = fmaf(db, vb, acc[m][1]);
                    }
                    __syncwarp();  // every lane has read the slot before it is refilled
                    async_issue(cur_half);
                    cur_half = cur_half + 1u == (uint32_t)H ? 0u : cur_half + 1u;
                }
            }
        } else if (tile_ok) {
#pragma unroll 1
            for (uint32_t ch0 = my_ks; ch0 < n_chunks; ch0 += ks * H) {
                if (cur_half == 0 || kSlots == 1) multiply_half(half0{}, ch0, acc);
                else if (cur_half == 1 || kSlots == 2) {
                    if constexpr (kSlots > 1) multiply_half(half1{}, ch0, acc);
                } else {
                    if constexpr (kSlots > 2) multiply_half(half2{}, ch0, acc);
                }
                cur_half = cur_half == (uint32_t)(kSlots - 1) ? 0u : cur_half + 1u;
            }
        }
        // ---- add the four lanes of each row, then the ks column splits ----
#pragma unroll
        for (int m = 0; m < M; ++m)
#pragma unroll
            for (int h = 0; h < 2; ++h) {
                float v = acc[m][h];
                v += __shfl_xor_sync(0xffffffffu, v, 1);
                v += __shfl_xor_sync(0xffffffffu, v, 2);
                acc[m][h] = v;
            }
        if (ks == 1) {
            if (tile_ok && t4 == 0) {
#pragma unroll
                for (int m = 0; m < M; ++m)
#pragma unroll
                    for (int h = 0; h < 2; ++h) {
                        const uint32_t row = tile * 16u + g + 8u * h;
                        if (row < rows) {
                            float *yp = a.y + (size_t)m * a.y_stride + row;
                            *yp = a.epilogue == TM_CUDA_EPI_ADD ? *yp + acc[m][h] : acc[m][h];
                        }
                    }
            }
        } else {
            __syncthreads();  // previous round's readers are done with `partial`
            if (t4 == 0) {
#pragma unroll
                for (int m = 0; m < M; ++m) {
                    partial[warp][m][g] = acc[m][0];
                    partial[warp][m][g + 8] = acc[m][1];
                }
            }
            __syncthreads();
            for (uint32_t i = threadIdx.x; i < tiles_per_cta * M * 16u; i += kThreads) {
                const uint32_t r16 = i & 15u, m = (i >> 4) % M, tl = i / (16u * M);
                const uint32_t row = (base + tl) * 16u + r16;
                if (base + tl < n_tiles && row < rows) {
                    float v = 0.0f;
                    for (uint32_t k = 0; k < ks; ++k) v += partial[tl * ks + k][m][r16];
                    float *yp = a.y + (size_t)m * a.y_stride + row;
                    *yp = a.epilogue == TM_CUDA_EPI_ADD ? *yp + v : v;
                }
            }
        }
    }
}

template <int M, int kSlots, int H, bool kAdd>
cudaError_t launch_gemv_form(tm_cuda_ctx *ctx, const gemv_args &a, int grid, size_t smem) {
    static std::atomic<bool> attr_set[64] = {};  // per device; contexts of a process share it
    const int dev = ctx->device;
    if (dev < 0 || dev >= 64 || !attr_set[dev].load(std::memory_order_acquire)) {
        cudaError_t e = cudaFuncSetAttribute(q8_gemv_kernel<M, kSlots, H, kAdd>,
                                             cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)ctx->smem_optin - 8192);
        if (e != cudaSuccess) return e;
        if (dev >= 0 && dev < 64) attr_set[dev].store(true, std::memory_order_release);
    }
    return tm_launch_pdl(ctx, q8_gemv_kernel<M, kSlots, H, kAdd>, dim3(grid), dim3(kThreads), smem, a);
}
template <int M, int kSlots, int H>
cudaError_t launch_gemv(tm_cuda_ctx *ctx, const gemv_args &a, int grid, size_t smem) {
    if constexpr (M == 1)
        if (a.add_p) return launch_gemv_form<M, kSlots, H, true>(ctx, a, grid, smem);
    return launch_gemv_form<M, kSlots, H, false>(ctx, a, grid, smem);
}

uint32_t digit_plane_bytes(uint32_t cols) {
    const uint32_t pad = (uint32_t)tm_round_up(cols, kChunkCols);
    return pad % 128u == 0 ? pad + 64u : pad;
}

// Resident CTAs per SM of the form the launcher picks for long column ranges: the register forms
// fit two; the shared-memory ring is limited by its shared memory (staged activations + 8 warps x 8
// slots + 1 KB the system reserves per CTA), at most four by registers.
uint32_t resident_ctas_per_sm(const tm_cuda_ctx *ctx, uint32_t cols, int m) {
    if (m != 1 || cols % 64u != 0u) return 2u;
    const size_t cta = (((size_t)token_smem(cols, digit_plane_bytes(cols)) + 15u) & ~(size_t)15u) +
                       (size_t)kWarps * 8u * 1088u + 1024u;
    if (cta - 1024u > ctx->smem_optin - 8192u) return 2u;
    const size_t fit = (228u * 1024u) / cta;
    return (uint32_t)(fit > 4u ? 4u : fit < 1u ? 1u : fit);
}

// One launch for `m` tokens (m in {1,2,4,8}) over a.rows rows.  The column split comes from the
// matrix shape alone, so small projections still fill the machine.
cudaError_t gemv_part(tm_cuda_ctx *ctx, gemv_args a, int m) {
    a.plane = digit_plane_bytes(a.cols);
    const size_t smem = (size_t)m * token_smem(a.cols, a.plane);
    const uint32_t n_tiles = (a.rows + 15u) / 16u;
    const uint32_t n_chunks = (a.cols + kChunkCols - 1u) / kChunkCols;
    // warps of one resident wave: the column split grows only while the grid stays within it
    // (taken from the one-token form whatever m is: the split must depend on the shape alone)
    const uint32_t want = (uint32_t)ctx->sm_count * resident_ctas_per_sm(ctx, a.cols, 1) * kWarps;
    // A row view takes the split of the matrix it is a view of, so that a row's partial sums are added
    // in the same order whether the whole matrix or a part of it is multiplied.
    const uint32_t shape_tiles = ((a.shape_rows ? a.shape_rows : a.rows) + 15u) / 16u;
    uint32_t ks = 1;
    while (ks < (uint32_t)kWarps && shape_tiles * ks * 2u <= want && ks * 2u <= n_chunks) ks <<= 1;
    a.ks = ks;
    const uint32_t tiles_per_cta = kWarps / ks;
    uint32_t ctas = (n_tiles + tiles_per_cta - 1u) / tiles_per_cta;
    if (ctas > 1u << 20) ctas = 1u << 20;  // the kernel strides over any remainder
    if (m > 1) {
        // Several tokens: staging them (norm, digit split) costs a CTA far more than streaming one row
        // tile's weights, so the grid is one resident wave and every warp walks its share of the tiles
        // with the activations staged once.  (Which CTA multiplies a tile does not change its sums.)
        const size_t fit = (size_t)ctx->smem_optin / (smem + 1024u);
        const uint32_t wave = (uint32_t)ctx->sm_count * (uint32_t)(fit >= 2u ? 2u : 1u);
        if (ctas > wave) ctas = wave;
    }
    switch (m) {
        case 8: return launch_gemv<8, 2, 2>(ctx, a, (int)ctas, smem);
        case 4: return launch_gemv<4, 2, 2>(ctx, a, (int)ctas, smem);
        case 2: return launch_gemv<2, 2, 2>(ctx, a, (int)ctas, smem);
        default:
            // Measured on the 8B-scale shapes and both lm_heads (same-box A/B): wherever a warp streams at
            // least six chunks per tile the shared-memory ring of eight chunks wins (64 registers, three
            // CTAs per SM, 192 KB of loads in flight per SM); it needs whole 64-column chunks, otherwise
            // one register slot of six chunks is next best; short column ranges do best with three
            // slots of two.
            if (n_chunks / ks >= 6u) {
                // Ring depth: 8 chunks per warp leaves room for three CTAs per SM; a grid that puts at
                // most one CTA on an SM anyway (the mid-size projections) takes the deepest ring that
                // fits instead, so that its few warps still keep enough bytes in flight.
                const size_t base = (smem + 15u) & ~(size_t)15u, budget = ctx->smem_optin - 8192u;
                auto ring_bytes = [&](int depth) { return base + (size_t)kWarps * (size_t)depth * 1088u; };
                if (a.cols % 64u == 0u && ring_bytes(8) <= budget) {
                    if (ctas <= (uint32_t)ctx->sm_count && n_chunks / ks >= 24u && ring_bytes(24) <= budget)
                        return launch_gemv<1, 0, 24>(ctx, a, (int)ctas, ring_bytes(24));
                    if (ctas <= (uint32_t)ctx->sm_count && n_chunks / ks >= 16u && ring_bytes(16) <= budget)
                        return launch_gemv<1, 0, 16>(ctx, a, (int)ctas, ring_bytes(16));
                    return launch_gemv<1, 0, 8>(ctx, a, (int)ctas, ring_bytes(8));
                }
                return launch_gemv<1, 1, 6>(ctx, a, (int)ctas, smem);
            }
            return launch_gemv<1, 3, 2>(ctx, a, (int)ctas, smem);
    }
}

// `m` tokens over the whole matrix.  A very tall matrix whose CTAs (8 row tiles each, no column
// split) do not fill a whole number of resident waves would spend up to a full CTA time on a nearly
// empty last wave (151936 rows: 4.01 waves).  Its rows are cut instead: the bulk that fills whole
// waves keeps ks = 1, the remaining rows go to a second launch that takes its own, much wider
// column split and slots into the SMs the bulk's last wave frees.  The cut depends on the shape
// only, so a (row, token) result is still the same for every batch size.
cudaError_t gemv_slice(tm_cuda_ctx *ctx, gemv_args a, int m) {
    a.y_stride = a.rows;
    const uint32_t per_sm = resident_ctas_per_sm(ctx, a.cols, 1);  // shape only, like the column split
    const uint32_t slots = (uint32_t)ctx->sm_count * per_sm;   // resident CTAs
    const uint32_t rows_per_cta = (uint32_t)kWarps * 16u;
    const uint32_t ctas = (a.rows + rows_per_cta - 1u) / rows_per_cta;
    const uint32_t rem = ctas % slots;
    if (ctas > 2u * slots && rem != 0u && rem * 2u < slots) {
        const uint32_t bulk_rows = (ctas - rem) * rows_per_cta;
        gemv_args bulk = a, rest = a;
        bulk.rows = bulk.shape_rows = bulk_rows;
        cudaError_t e = gemv_part(ctx, bulk, m);
        if (e != cudaSuccess) return e;
        rest.q = a.q + (size_t)bulk_rows * a.cols;
        rest.d = a.d + (size_t)bulk_rows * (a.cols / 32u);
        rest.y = a.y + bulk_rows;
        rest.rows = rest.shape_rows = a.rows - bulk_rows;
        return gemv_part(ctx, rest, m);
    }
    return gemv_part(ctx, a, m);
}

// Whole batch in slices of 8/4/2/1 tokens that fit shared memory.
int gemv_batch(tm_cuda_ctx *ctx, gemv_args a, uint32_t batch, uint64_t *kernels, char *err,
               size_t err_cap) {
    const size_t per_token = token_smem(a.cols, digit_plane_bytes(a.cols));
    const size_t budget = ctx->smem_optin - 16384;
    if (per_token > budget)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "cols %u exceeds the activation stage of one CTA (%zu bytes)", a.cols, budget);
    uint32_t done = 0;
    while (done < batch) {
        int m = 8;
        while (m > 1 && ((uint32_t)m > batch - done || (size_t)m * per_token > budget)) m >>= 1;
        gemv_args s = a;
        s.x = a.x + (size_t)done * a.cols;
        s.y = a.y + (size_t)done * a.rows;
        if (a.prologue == TM_CUDA_PRO_SILU_MUL || a.prologue == TM_CUDA_PRO_GELU_MUL)
            s.pro = a.pro + (size_t)done * a.cols;
        cudaError_t e = gemv_slice(ctx, s, m);
        if (e != cudaSuccess)
            return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "Q8_0 GEMV launch failed: %s",
                           cudaGetErrorString(e));
        *kernels += 1;
        done += (uint32_t)m;
    }
    return TM_CUDA_OK;
}

// ---- repacking --------------------------------------------------------------

// One thread per (row, block): 34 raw bytes -> 32 quants + 1 scale.
__global__ void q8_pack_kernel(const unsigned char *raw, signed char *q, __half *d, uint32_t cols,
                               uint32_t row0, uint32_t nrows) {
    const uint32_t nb = cols / 32u;
    const size_t total = (size_t)nrows * nb;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / nb), b = (uint32_t)(i % nb);
        const unsigned short *src = (const unsigned short *)(raw + i * 34);  // 2-byte aligned
        unsigned short h[17];
#pragma unroll
        for (int k = 0; k < 17; ++k) h[k] = src[k];
        ((unsigned short *)d)[(size_t)(row0 + r) * nb + b] = h[0];
        uint32_t *dst = (uint32_t *)(q + (size_t)(row0 + r) * cols + (size_t)b * 32);
#pragma unroll
        for (int k = 0; k < 8; ++k) dst[k] = (uint32_t)h[1 + 2 * k] | ((uint32_t)h[2 + 2 * k] << 16);
    }
}

__global__ void q8_unpack_kernel(unsigned char *raw, const signed char *q, const __half *d,
                                 uint32_t cols, uint32_t row0, uint32_t nrows) {
    const uint32_t nb = cols / 32u;
    const size_t total = (size_t)nrows * nb;
    for (size_t i = (size_t)blockIdx.x * blockDim.x + threadIdx.x; i < total;
         i += (size_t)gridDim.x * blockDim.x) {
        const uint32_t r = (uint32_t)(i / nb), b = (uint32_t)(i % nb);
        unsigned short *dst = (unsigned short *)(raw + i * 34);
        dst[0] = ((const unsigned short *)d)[(size_t)(row0 + r) * nb + b];
        const unsigned short *src = (const unsigned short *)(q + (size_t)(row0 + r) * cols + (size_t)b * 32);
#pragma unroll
        for (int k = 0; k < 16; ++k) dst[1 + k] = src[k];
    }
}

// out[c] = d(row, c/32) * q(row, c), c < cols; row < 0 writes zeros.
__device__ __forceinline__ void dequant_row(const signed char *q, const __half *d, uint32_t cols,
                                            long row, float scale, float *out) {
    const uint32_t nb = cols / 32u;
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x) {
        float v = 0.0f;
        if (row >= 0) {
            v = __half2float(d[(size_t)row * nb + c / 32u]) * (float)q[(size_t)row * cols + c];
            if (scale != 0.0f) v *= scale;
        }
        out[c] = v;
    }
}

__global__ void q8_row_kernel(const signed char *q, const __half *d, uint32_t cols, uint32_t row,
                              float *out) {
    dequant_row(q, d, cols, (long)row, 0.0f, out);
}

__global__ void q8_row_indirect_kernel(const signed char *q, const __half *d, uint32_t rows,
                                       uint32_t cols, const uint32_t *ids, uint32_t slot,
                                       const uint32_t *pos, int bias, uint32_t ids_len, float scale,
                                       float *out) {
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    uint32_t s = slot;
    if (pos) s = slot + *pos + (uint32_t)bias;
    long row = -1;
    if (s < ids_len) {
        const uint32_t id = ids[s];
        if (id < rows) row = (long)id;
    }
    dequant_row(q, d, cols, row, scale, out);
}

// out[t][c] = dequant(row ids[first + t])[c] (* scale), t < n; ids outside the table write zeros.
__global__ void q8_rows_gather_kernel(const signed char *q, const __half *d, uint32_t rows, uint32_t cols,
                                      const uint32_t *ids, uint32_t first, float scale, float *out) {
    const uint32_t t = blockIdx.y, nb = cols / 32u;
    const uint32_t id = ids[first + t];
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x) {
        float v = 0.0f;
        if (id < rows) {
            v = __half2float(d[(size_t)id * nb + c / 32u]) * (float)q[(size_t)id * cols + c];
            if (scale != 0.0f) v *= scale;
        }
        out[(size_t)t * cols + c] = v;
    }
}

// One row per sequence: out[s] = row ids[s * stride + pos[s] + bias] (zeros when the slot or the id is outside).
__global__ void q8_rows_gather_seq_kernel(const signed char *q, const __half *d, uint32_t rows, uint32_t cols,
                                          const uint32_t *ids, uint32_t stride, const uint32_t *pos, int bias,
                                          float scale, float *out) {
    tmdev::pdl_trigger();
    tmdev::pdl_wait();
    const uint32_t t = blockIdx.y, nb = cols / 32u;
    const uint32_t slot = pos[t] + (uint32_t)bias;
    const uint32_t id = slot < stride ? ids[(size_t)t * stride + slot] : 0xFFFFFFFFu;
    for (uint32_t c = blockIdx.x * blockDim.x + threadIdx.x; c < cols; c += gridDim.x * blockDim.x) {
        float v = 0.0f;
        if (id < rows) {
            v = __half2float(d[(size_t)id * nb + c / 32u]) * (float)q[(size_t)id * cols + c];
            if (scale != 0.0f) v *= scale;
        }
        out[(size_t)t * cols + c] = v;
    }
}

}  // namespace

extern "C" {

size_t tm_cuda_q8_0_packed_bytes(uint32_t rows, uint32_t cols) {
    if (rows == 0 || cols == 0 || cols % 32 != 0) return 0;
    return tm_q8_qplane_bytes(rows, cols) + (size_t)rows * (cols / 32) * 2;
}

int tm_cuda_q8_0_pack(tm_cuda_ctx *ctx, tm_cuda_buffer *dst, uint32_t rows, uint32_t cols,
                      tm_cuda_buffer *raw, size_t raw_off, uint32_t row0, uint32_t nrows,
                      char *err, size_t err_cap) {
    TM_ENTER();
    if (rows == 0 || cols == 0 || cols % 32 != 0 || nrows == 0 || row0 >= rows || nrows > rows - row0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "pack of rows [%u, +%u) of a %u x %u Q8_0 matrix is out of range", row0, nrows,
                       rows, cols);
    if (raw_off % 2 != 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "raw offset must be even");
    TM_CHECK_BUF(dst, tm_cuda_q8_0_packed_bytes(rows, cols), "packed matrix");
    TM_CHECK_BUF(raw, raw_off + (size_t)nrows * (cols / 32) * 34, "raw rows");
    if (dst->parent)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "a packed matrix must own its buffer");
    if (dst->layout == TM_LAYOUT_Q8_0_PACKED && (dst->rows != rows || dst->cols != cols))
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "buffer already holds a packed %u x %u matrix", dst->rows, dst->cols);
    TM_OP_BEGIN("q8_0_pack");
    const size_t total = (size_t)nrows * (cols / 32);
    const int grid = (int)((total + 255) / 256 > 65535 ? 65535 : (total + 255) / 256);
    q8_pack_kernel<<<grid, 256, 0, ctx->stream>>>(
        raw->dev + raw_off, (signed char *)dst->dev,
        (__half *)(dst->dev + tm_q8_qplane_bytes(rows, cols)), cols, row0, nrows);
    dst->layout = TM_LAYOUT_Q8_0_PACKED;
    dst->rows = rows;
    dst->cols = cols;
    dst->qp = dst->dev;
    dst->dp = dst->dev + tm_q8_qplane_bytes(rows, cols);
    TM_OP_END(1);
}

tm_cuda_buffer *tm_cuda_q8_0_row_view(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows,
                                      uint32_t cols, uint32_t row0, uint32_t nrows, char *err,
                                      size_t err_cap) {
    if (!ctx) {
        tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "null context");
        return nullptr;
    }
    std::lock_guard<std::mutex> lock(ctx->mu);
    if (tm_check_packed(ctx, w, rows, cols, err, err_cap) != TM_CUDA_OK) return nullptr;
    if (nrows == 0 || row0 >= rows || nrows > rows - row0) {
        tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "row view [%u, +%u) of a %u-row matrix", row0, nrows, rows);
        return nullptr;
    }
    tm_cuda_buffer *b = new tm_cuda_buffer();
    b->owner = ctx;
    b->parent = w;
    b->dev = w->dev;
    b->len = w->len;
    b->layout = TM_LAYOUT_Q8_0_PACKED;
    b->rows = nrows;
    b->cols = cols;
    b->qp = w->qp + (size_t)row0 * cols;
    b->dp = w->dp + (size_t)row0 * (cols / 32) * 2;
    w->views += 1;
    ctx->live.insert(b);
    return b;
}

int tm_cuda_q8_0_unpack(tm_cuda_ctx *ctx, tm_cuda_buffer *src, uint32_t rows, uint32_t cols,
                        tm_cuda_buffer *raw, size_t raw_off, uint32_t row0, uint32_t nrows,
                        char *err, size_t err_cap) {
    TM_ENTER();
    int rc = tm_check_packed(ctx, src, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    if (nrows == 0 || row0 >= rows || nrows > rows - row0 || raw_off % 2 != 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "unpack row range out of bounds");
    TM_CHECK_BUF(raw, raw_off + (size_t)nrows * (cols / 32) * 34, "raw rows");
    TM_OP_BEGIN("q8_0_unpack");
    const size_t total = (size_t)nrows * (cols / 32);
    const int grid = (int)((total + 255) / 256 > 65535 ? 65535 : (total + 255) / 256);
    q8_unpack_kernel<<<grid, 256, 0, ctx->stream>>>(
        raw->dev + raw_off, (const signed char *)src->qp, (const __half *)src->dp, cols, row0, nrows);
    TM_OP_END(1);
}

static int gemv_common(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y,
                       uint32_t rows, uint32_t cols, uint32_t batch, uint32_t x_off, uint32_t y_off,
                       int prologue, tm_cuda_buffer *pro, float eps, int epilogue, const char *label,
                       char *err, size_t err_cap) {
    int rc = tm_check_packed(ctx, w, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    if (batch == 0 || batch > TM_CUDA_GEMM_MAX_BATCH)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "batch %u outside 1..%u", batch,
                       TM_CUDA_GEMM_MAX_BATCH);
    TM_CHECK_BUF(x, ((size_t)x_off + (size_t)batch * cols) * 4, "activation");
    TM_CHECK_BUF(y, ((size_t)y_off + (size_t)batch * rows) * 4, "output");
    if (prologue < TM_CUDA_PRO_NONE || prologue > TM_CUDA_PRO_GELU_MUL ||
        (epilogue != TM_CUDA_EPI_STORE && epilogue != TM_CUDA_EPI_ADD))
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "unknown prologue/epilogue");
    if (prologue == TM_CUDA_PRO_RMSNORM) TM_CHECK_BUF(pro, (size_t)cols * 4, "norm weight");
    if (prologue == TM_CUDA_PRO_SILU_MUL || prologue == TM_CUDA_PRO_GELU_MUL)
        TM_CHECK_BUF(pro, (size_t)batch * cols * 4, "gate multiplicand");
    gemv_args a;
    a.q = (const signed char *)w->qp;
    a.d = (const __half *)w->dp;
    a.x = (const float *)x->dev + x_off;
    a.y = (float *)y->dev + y_off;
    a.pro = pro ? (const float *)pro->dev : nullptr;
    a.rows = rows;
    a.cols = cols;
    a.shape_rows = rows;
    for (const tm_cuda_buffer *p = w->parent; p && p->layout == TM_LAYOUT_Q8_0_PACKED; p = p->parent) a.shape_rows = p->rows;
    a.eps = eps;
    a.prologue = prologue;
    a.epilogue = epilogue;
    if (ctx->program)
        return tm_step_record_gemv(ctx, a.q, a.d, a.x, a.y, a.pro, rows, cols, prologue, epilogue, eps, batch, err, err_cap);
    TM_OP_BEGIN(label);
    uint64_t kernels = 0;
    rc = gemv_batch(ctx, a, batch, &kernels, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    TM_OP_END(kernels);
}

int tm_cuda_q8_0_gemv(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y,
                      uint32_t rows, uint32_t cols, char *err, size_t err_cap) {
    TM_ENTER();
    return gemv_common(ctx, w, x, y, rows, cols, 1, 0, 0, TM_CUDA_PRO_NONE, nullptr, 0.0f,
                       TM_CUDA_EPI_STORE, "q8_0_gemv", err, err_cap);
}

int tm_cuda_q8_0_gemm(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y,
                      uint32_t rows, uint32_t cols, uint32_t batch, uint32_t x_off, uint32_t y_off,
                      char *err, size_t err_cap) {
    TM_ENTER();
    return gemv_common(ctx, w, x, y, rows, cols, batch, x_off, y_off, TM_CUDA_PRO_NONE, nullptr,
                       0.0f, TM_CUDA_EPI_STORE, "q8_0_gemm", err, err_cap);
}

int tm_cuda_q8_0_gemv_fused(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x,
                            tm_cuda_buffer *y, uint32_t rows, uint32_t cols, int prologue,
                            tm_cuda_buffer *pro, float eps, int epilogue, char *err,
                            size_t err_cap) {
    TM_ENTER();
    return gemv_common(ctx, w, x, y, rows, cols, 1, 0, 0, prologue, pro, eps, epilogue,
                       "q8_0_gemv_fused", err, err_cap);
}

int tm_cuda_q8_0_gemv_addnorm(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *add_p,
                              tm_cuda_buffer *add_w, tm_cuda_buffer *x_out, tm_cuda_buffer *norm_w, tm_cuda_buffer *y,
                              uint32_t rows, uint32_t cols, float eps, char *err, size_t err_cap) {
    TM_ENTER();
    int rc = tm_check_packed(ctx, w, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    if (cols > (uint32_t)(kThreads * 16))
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "cols %u above the %d this form stages in one pass", cols,
                       kThreads * 16);
    TM_CHECK_BUF(x, (size_t)cols * 4, "x");
    TM_CHECK_BUF(add_p, (size_t)cols * 4, "vector to add");
    TM_CHECK_BUF(add_w, (size_t)cols * 4, "its norm weight");
    TM_CHECK_BUF(x_out, (size_t)cols * 4, "x output");
    TM_CHECK_BUF(norm_w, (size_t)cols * 4, "norm weight");
    TM_CHECK_BUF(y, (size_t)rows * 4, "output");
    if (x_out == x || x_out->dev == x->dev)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "x_out must be a buffer other than x (every CTA reads x)");
    if (ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "operator q8_0_gemv_addnorm cannot be recorded into a persistent program");
    gemv_args a;
    a.q = (const signed char *)w->qp;
    a.d = (const __half *)w->dp;
    a.x = (const float *)x->dev;
    a.y = (float *)y->dev;
    a.pro = (const float *)norm_w->dev;
    a.rows = rows;
    a.cols = cols;
    a.shape_rows = rows;
    for (const tm_cuda_buffer *p = w->parent; p && p->layout == TM_LAYOUT_Q8_0_PACKED; p = p->parent) a.shape_rows = p->rows;
    a.eps = eps;
    a.prologue = TM_CUDA_PRO_RMSNORM;
    a.epilogue = TM_CUDA_EPI_STORE;
    a.add_p = (const float *)add_p->dev;
    a.add_w = (const float *)add_w->dev;
    a.x_out = (float *)x_out->dev;
    TM_OP_BEGIN("q8_0_gemv_addnorm");
    uint64_t kernels = 0;
    rc = gemv_batch(ctx, a, 1, &kernels, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    TM_OP_END(kernels);
}

int tm_cuda_q8_0_gemm_fused(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t rows,
                            uint32_t cols, uint32_t batch, int prologue, tm_cuda_buffer *pro, float eps, int epilogue,
                            char *err, size_t err_cap) {
    TM_ENTER();
    if (ctx->program && batch != 1)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "operator q8_0_gemm_fused cannot be recorded into a persistent program");
    return gemv_common(ctx, w, x, y, rows, cols, batch, 0, 0, prologue, pro, eps, epilogue, "q8_0_gemm_fused", err,
                       err_cap);
}

int tm_cuda_q8_0_row_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *out, uint32_t row,
                         uint32_t cols, uint32_t out_off, char *err, size_t err_cap) {
    TM_ENTER();
    if (!w || ctx->live.find(w) == ctx->live.end() || w->layout != TM_LAYOUT_Q8_0_PACKED ||
        w->cols != cols)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "weight buffer is not a packed Q8_0 matrix of %u columns", cols);
    if (row >= w->rows)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "row %u outside the %u rows", row, w->rows);
    TM_CHECK_BUF(out, ((size_t)out_off + cols) * 4, "row output");
    TM_OP_BEGIN("q8_0_row");
    q8_row_kernel<<<(cols + 255) / 256, 256, 0, ctx->stream>>>(
        (const signed char *)w->qp, (const __half *)w->dp, cols, row, (float *)out->dev + out_off);
    TM_OP_END(1);
}

static int row_indirect(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols,
                        tm_cuda_buffer *ids, uint32_t slot, tm_cuda_buffer *pos_buf,
                        uint32_t pos_index, int32_t bias, float scale, tm_cuda_buffer *out,
                        char *err, size_t err_cap) {
    int rc = tm_check_packed(ctx, w, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    TM_CHECK_BUF(ids, ((size_t)slot + 1) * 4, "token ids");
    TM_CHECK_BUF(out, (size_t)cols * 4, "row output");
    const uint32_t *pos = nullptr;
    if (pos_buf) {
        TM_CHECK_BUF(pos_buf, ((size_t)pos_index + 1) * 4, "position");
        pos = (const uint32_t *)pos_buf->dev + pos_index;
    }
    if (ctx->program)
        return tm_step_record_embed(ctx, w->qp, w->dp, rows, cols, (const uint32_t *)ids->dev, slot, pos, (int)bias,
                                    (uint32_t)(ids->len / 4), scale, (float *)out->dev, err, err_cap);
    TM_OP_BEGIN("row_indirect");
    TM_CUDA_TRY(tm_launch_pdl(ctx, q8_row_indirect_kernel, dim3((cols + 255) / 256), dim3(256), 0,
                              (const signed char *)w->qp, (const __half *)w->dp, rows, cols,
                              (const uint32_t *)ids->dev, slot, pos, (int)bias, (uint32_t)(ids->len / 4), scale,
                              (float *)out->dev));
    TM_OP_END(1);
}

int tm_cuda_row_indirect_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t type_id, uint32_t rows,
                             uint32_t cols, tm_cuda_buffer *ids, uint32_t slot,
                             tm_cuda_buffer *out, char *err, size_t err_cap) {
    TM_ENTER();
    if (type_id != 8)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED,
                       "row_indirect supports Q8_0 (type 8) matrices; got type %u", type_id);
    return row_indirect(ctx, w, rows, cols, ids, slot, nullptr, 0, 0, 0.0f, out, err, err_cap);
}

int tm_cuda_rows_indirect_f32(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols,
                              tm_cuda_buffer *ids, uint32_t first, uint32_t n, float scale,
                              tm_cuda_buffer *out, char *err, size_t err_cap) {
    TM_ENTER();
    int rc = tm_check_packed(ctx, w, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    if (n == 0 || n > 65535u) return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "row count %u outside 1..65535", n);
    TM_CHECK_BUF(ids, ((size_t)first + n) * 4, "token ids");
    TM_CHECK_BUF(out, (size_t)n * cols * 4, "rows output");
    TM_OP_BEGIN("rows_indirect");
    q8_rows_gather_kernel<<<dim3((cols + 255) / 256, n), 256, 0, ctx->stream>>>(
        (const signed char *)w->qp, (const __half *)w->dp, rows, cols, (const uint32_t *)ids->dev, first,
        scale, (float *)out->dev);
    TM_OP_END(1);
}

int tm_cuda_rows_indirect_seq_f32_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols,
                                      tm_cuda_buffer *ids, uint32_t ids_stride, tm_cuda_buffer *pos_buf,
                                      uint32_t n_seq, int32_t bias, float scale, tm_cuda_buffer *out, char *err,
                                      size_t err_cap) {
    TM_ENTER();
    int rc = tm_check_packed(ctx, w, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    if (n_seq == 0 || n_seq > 65535u || ids_stride == 0)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "%u sequences with logs of %u slots", n_seq, ids_stride);
    TM_CHECK_BUF(ids, (size_t)n_seq * ids_stride * 4, "token logs");
    TM_CHECK_BUF(pos_buf, (size_t)n_seq * 4, "positions");
    TM_CHECK_BUF(out, (size_t)n_seq * cols * 4, "rows output");
    if (ctx->program)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "operator rows_indirect_seq cannot be recorded into a persistent program");
    TM_OP_BEGIN("rows_indirect_seq");
    TM_CUDA_TRY(tm_launch_pdl(ctx, q8_rows_gather_seq_kernel, dim3((cols + 255) / 256, n_seq), dim3(256), 0,
                              (const signed char *)w->qp, (const __half *)w->dp, rows, cols, (const uint32_t *)ids->dev,
                              ids_stride, (const uint32_t *)pos_buf->dev, (int)bias, scale, (float *)out->dev));
    TM_OP_END(1);
}

int tm_cuda_row_indirect_f32_dev(tm_cuda_ctx *ctx, tm_cuda_buffer *w, uint32_t rows, uint32_t cols,
                                 tm_cuda_buffer *ids, uint32_t base, tm_cuda_buffer *pos_buf,
                                 uint32_t pos_index, int32_t bias, float scale,
                                 tm_cuda_buffer *out, char *err, size_t err_cap) {
    TM_ENTER();
    if (!pos_buf) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "null position buffer");
    return row_indirect(ctx, w, rows, cols, ids, base, pos_buf, pos_index, bias, scale, out, err,
                        err_cap);
}

}  // extern "C"
