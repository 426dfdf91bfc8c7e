// Prefill attention on the tensor cores, tolerance-qualified.
//
// Same contract as the chunk attention operator (native/metal/tm_metal.h:367,
// native/metal/kernels.metal: query row t of a chunk at pos0 attends keys
// [start, pos0 + t], start = seq > window ? seq - window : 0, softmax over
// q.k * scale, f16 K/V cache) but not its arithmetic order: Q and the softmax
// weights are rounded to binary16 and multiplied with mma.sync (m16n8k16, f32
// accumulate), keys are visited in tiles of 64 with a running maximum.  The
// engine uses it unless `exact` is asked; the blockwise kernel stays the
// bit-identical form.  Attention is not the Q8_0 hot path: this kernel exists
// because a 512-token prefill otherwise spends half its time here.
//
// One CTA of 4 warps serves 64 queries of one head (16 per warp) and, when the
// head dim exceeds 128, one 128-wide half of the value dims (grid.z).
#include "tm_cuda_internal.cuh"

namespace {

constexpr int kBQ = 64, kBKV = 64, kThreads = 128;

__device__ __forceinline__ uint32_t smem_u32(const void *p) { return (uint32_t)__cvta_generic_to_shared(p); }

// Byte offset of 16-byte chunk `chunk` of row `row` in a tile of PITCH-byte rows, XOR-swizzled so
// that the eight rows an ldmatrix touches fall into distinct bank groups.
template <int PITCH>
__device__ __forceinline__ uint32_t sw(uint32_t row, uint32_t chunk) {
    if (PITCH >= 128) return row * PITCH + ((chunk ^ (row & 7u)) << 4);
    return row * PITCH + ((chunk ^ ((row >> 1) & 3u)) << 4);  // 64-byte rows: two rows per 128 bytes
}

__device__ __forceinline__ void ldsm_x4(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void ldsm_x4_t(uint32_t addr, uint32_t &r0, uint32_t &r1, uint32_t &r2, uint32_t &r3) {
    asm volatile("ldmatrix.sync.aligned.m8n8.x4.trans.shared.b16 {%0,%1,%2,%3}, [%4];"
                 : "=r"(r0), "=r"(r1), "=r"(r2), "=r"(r3)
                 : "r"(addr));
}
__device__ __forceinline__ void mma_f16(float (&d)[4], uint32_t a0, uint32_t a1, uint32_t a2, uint32_t a3, uint32_t b0,
                                        uint32_t b1) {
    asm volatile(
        "mma.sync.aligned.m16n8k16.row.col.f32.f16.f16.f32 {%0,%1,%2,%3}, {%4,%5,%6,%7}, {%8,%9}, {%0,%1,%2,%3};"
        : "+f"(d[0]), "+f"(d[1]), "+f"(d[2]), "+f"(d[3])
        : "r"(a0), "r"(a1), "r"(a2), "r"(a3), "r"(b0), "r"(b1));
}
__device__ __forceinline__ void cp_async16(uint32_t dst, const void *src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"(dst), "l"(src) : "memory");
}
__device__ __forceinline__ uint32_t pack_h2(float a, float b) {
    const __half2 h = __floats2half2_rn(a, b);
    return *(const uint32_t *)&h;
}

struct attn_args {
    const float *q;    // [n][heads][HD]
    const __half *kc;  // [kv_heads][cap][HD]
    const __half *vc;
    float *out;        // [n][heads][HD]
    uint32_t heads, group, pos0, cap, n, window;
    float scale_log2e;
};

template <int HD>
struct attn_cfg {
    static constexpr int kDV = HD > 128 ? 128 : HD;      // value dims per CTA
    static constexpr int kQPitch = HD * 2, kVPitch = kDV * 2;
    static constexpr uint32_t kQBytes = kBQ * kQPitch, kKBytes = kBKV * kQPitch, kVBytes = kBKV * kVPitch;
    static constexpr uint32_t kStage = kKBytes + kVBytes;
    static constexpr uint32_t kBytes = kQBytes + 2 * kStage;
};

template <int HD>
__global__ void __launch_bounds__(kThreads) attention_chunk_mma_kernel(const attn_args a) {
    using C = attn_cfg<HD>;
    constexpr int DV = C::kDV;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *sQ = smem, *sKV = smem + C::kQBytes;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t head = blockIdx.y, kvh = head / a.group;
    const uint32_t q0 = blockIdx.x * kBQ;        // first query (chunk row) of this CTA
    const uint32_t dv0 = blockIdx.z * DV;        // first value dim of this CTA
    const uint32_t q_last = min(q0 + kBQ, a.n) - 1u;
    // Keys any query of the block may see: from the first query's window start to the last query's position.
    const uint32_t seq_first = a.pos0 + q0 + 1u;
    const uint32_t kv_lo = (a.window != 0u && seq_first > a.window) ? seq_first - a.window : 0u;
    const uint32_t kv_hi = a.pos0 + q_last;  // inclusive
    const uint32_t tile_lo = kv_lo / kBKV, tile_hi = kv_hi / kBKV;
    const __half *kp = a.kc + (size_t)kvh * a.cap * HD, *vp = a.vc + (size_t)kvh * a.cap * HD;

    auto load_tile = [&](uint32_t tile, int stage) {
        unsigned char *sK = sKV + stage * C::kStage, *sV = sK + C::kKBytes;
        const uint32_t j0 = tile * kBKV;
        constexpr int KCH = HD / 8, VCH = DV / 8;  // 16-byte chunks per row
        for (int i = tid; i < kBKV * KCH; i += kThreads) {
            const uint32_t r = i / KCH, c = i % KCH;
            const uint32_t j = min(j0 + r, kv_hi);  // rows past the last visible key repeat it (they are masked)
            cp_async16(smem_u32(sK) + sw<C::kQPitch>(r, c), kp + (size_t)j * HD + c * 8);
        }
        for (int i = tid; i < kBKV * VCH; i += kThreads) {
            const uint32_t r = i / VCH, c = i % VCH;
            const uint32_t j = min(j0 + r, kv_hi);
            cp_async16(smem_u32(sV) + sw<C::kVPitch>(r, c), vp + (size_t)j * HD + dv0 + c * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };

    load_tile(tile_lo, 0);
    // Q: f32 -> f16 into the swizzled tile (rows past the chunk are zero).
    for (int i = tid; i < kBQ * (HD / 8); i += kThreads) {
        const uint32_t r = i / (HD / 8), c = i % (HD / 8);
        uint4 w = make_uint4(0, 0, 0, 0);
        if (q0 + r < a.n) {
            const float *src = a.q + ((size_t)(q0 + r) * a.heads + head) * HD + c * 8;
            const float4 f0 = *(const float4 *)src, f1 = *(const float4 *)(src + 4);
            w = make_uint4(pack_h2(f0.x, f0.y), pack_h2(f0.z, f0.w), pack_h2(f1.x, f1.y), pack_h2(f1.z, f1.w));
        }
        *(uint4 *)(sQ + sw<C::kQPitch>(r, c)) = w;
    }

    float o[DV / 8][4];
#pragma unroll
    for (int i = 0; i < DV / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run[2] = {-INFINITY, -INFINITY}, l_run[2] = {0.0f, 0.0f};
    // Query rows of this thread: warp*16 + g and + 8; their positions and window starts.
    uint32_t qpos[2], qstart[2];
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t qi = q0 + warp * 16 + g + 8 * h;
        qpos[h] = a.pos0 + qi;
        const uint32_t seq = qpos[h] + 1u;
        qstart[h] = (a.window != 0u && seq > a.window) ? seq - a.window : 0u;
        if (qi >= a.n) qstart[h] = 0xffffffffu;  // a row past the chunk sees nothing
    }

    for (uint32_t tile = tile_lo; tile <= tile_hi; ++tile) {
        const int stage = (int)((tile - tile_lo) & 1u);
        if (tile < tile_hi) {
            load_tile(tile + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();
        const uint32_t sK = smem_u32(sKV + stage * C::kStage), sV = sK + C::kKBytes;

        // ---- S = Q K^T for 16 queries x 64 keys ----
        float s[kBKV / 8][4];
#pragma unroll
        for (int i = 0; i < kBKV / 8; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
        for (int kt = 0; kt < HD / 16; ++kt) {
            uint32_t a0, a1, a2, a3;
            {
                const uint32_t m = lane >> 3;
                const uint32_t row = warp * 16 + (m & 1u) * 8 + (lane & 7), chunk = kt * 2 + (m >> 1);
                ldsm_x4(smem_u32(sQ) + sw<C::kQPitch>(row, chunk), a0, a1, a2, a3);
            }
#pragma unroll
            for (int np = 0; np < kBKV / 16; ++np) {  // two key n-tiles per ldmatrix
                uint32_t b0, b1, b2, b3;
                const uint32_t m = lane >> 3;
                const uint32_t row = np * 16 + (m >> 1) * 8 + (lane & 7), chunk = kt * 2 + (m & 1u);
                ldsm_x4(sK + sw<C::kQPitch>(row, chunk), b0, b1, b2, b3);
                mma_f16(s[2 * np], a0, a1, a2, a3, b0, b1);
                mma_f16(s[2 * np + 1], a0, a1, a2, a3, b2, b3);
            }
        }
        // ---- mask, running maximum, exponentials ----
        const uint32_t j0 = tile * kBKV;
        float mx[2] = {-INFINITY, -INFINITY};
#pragma unroll
        for (int i = 0; i < kBKV / 8; ++i)
#pragma unroll
            for (int e = 0; e < 4; ++e) {
                const int h = e >> 1;
                const uint32_t j = j0 + i * 8 + 2 * t + (e & 1);
                const bool vis = j <= qpos[h] && j >= qstart[h] && qstart[h] != 0xffffffffu;
                s[i][e] = vis ? s[i][e] * a.scale_log2e : -INFINITY;
                mx[h] = fmaxf(mx[h], s[i][e]);
            }
        float alpha[2], m_use[2];
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 1));
            mx[h] = fmaxf(mx[h], __shfl_xor_sync(0xffffffffu, mx[h], 2));
            const float m_new = fmaxf(m_run[h], mx[h]);
            m_use[h] = m_new == -INFINITY ? 0.0f : m_new;  // nothing visible yet: every weight is exp2(-inf) = 0
            alpha[h] = exp2f(m_run[h] - m_use[h]);         // m_run = -inf gives 0
            m_run[h] = m_new;
        }
        float rs[2] = {0.0f, 0.0f};
        uint32_t pa[kBKV / 16][4];  // the weights as A fragments of the second product
#pragma unroll
        for (int i = 0; i < kBKV / 8; ++i) {
            const float p0 = exp2f(s[i][0] - m_use[0]), p1 = exp2f(s[i][1] - m_use[0]);
            const float p2 = exp2f(s[i][2] - m_use[1]), p3 = exp2f(s[i][3] - m_use[1]);
            rs[0] += p0 + p1;
            rs[1] += p2 + p3;
            pa[i >> 1][(i & 1) * 2] = pack_h2(p0, p1);      // rows g:   a0a1 (keys 0-7) / a4a5 (keys 8-15)
            pa[i >> 1][(i & 1) * 2 + 1] = pack_h2(p2, p3);  // rows g+8: a2a3 / a6a7
        }
#pragma unroll
        for (int h = 0; h < 2; ++h) {
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 1);
            rs[h] += __shfl_xor_sync(0xffffffffu, rs[h], 2);
            l_run[h] = l_run[h] * alpha[h] + rs[h];
        }
#pragma unroll
        for (int i = 0; i < DV / 8; ++i) {
            o[i][0] *= alpha[0];
            o[i][1] *= alpha[0];
            o[i][2] *= alpha[1];
            o[i][3] *= alpha[1];
        }
        // ---- O += P V ----
#pragma unroll
        for (int kk = 0; kk < kBKV / 16; ++kk) {
#pragma unroll
            for (int dp = 0; dp < DV / 16; ++dp) {  // two dim n-tiles per ldmatrix
                uint32_t b0, b1, b2, b3;
                const uint32_t m = lane >> 3;
                const uint32_t row = kk * 16 + (m & 1u) * 8 + (lane & 7), chunk = dp * 2 + (m >> 1);
                ldsm_x4_t(sV + sw<C::kVPitch>(row, chunk), b0, b1, b2, b3);
                mma_f16(o[2 * dp], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b0, b1);
                mma_f16(o[2 * dp + 1], pa[kk][0], pa[kk][1], pa[kk][2], pa[kk][3], b2, b3);
            }
        }
        __syncthreads();  // the stage is refilled by the next iteration's prefetch
    }
    // ---- normalise and store ----
#pragma unroll
    for (int h = 0; h < 2; ++h) {
        const uint32_t qi = q0 + warp * 16 + g + 8 * h;
        if (qi >= a.n) continue;
        const float inv = 1.0f / l_run[h];
        float *dst = a.out + ((size_t)qi * a.heads + head) * HD + dv0 + 2 * t;
#pragma unroll
        for (int i = 0; i < DV / 8; ++i)
            *(float2 *)(dst + i * 8) = make_float2(o[i][2 * h] * inv, o[i][2 * h + 1] * inv);
    }
}

// Per-head RMS norm of q and k, split-half RoPE at pos0 + t, f16 K/V store: the four launches that
// precede chunk attention (rmsnorm x2, rope, kv_store) as one.  One warp per (token, vector),
// vectors = query heads, then KV heads; q is normed and rotated in place, k is normed, rotated and
// written to the cache together with v (k itself is left as it was).  Warp-shuffle sum of squares,
// so the low bits differ from the one-CTA-per-row norm: part of the tolerance-qualified prefill.
__global__ void __launch_bounds__(256) qk_prep_chunk_kernel(float *q, const float *k, const float *v,
                                                             const float *q_norm, const float *k_norm,
                                                             const float *inv_freq, __half *kc, __half *vc,
                                                             uint32_t heads, uint32_t kvh, uint32_t hd, uint32_t n_rot,
                                                             uint32_t pos0, uint32_t cap, uint32_t n, float eps) {
    const uint32_t lane = threadIdx.x & 31u;
    const uint32_t vec = blockIdx.x * 8u + (threadIdx.x >> 5), per_tok = heads + kvh;
    if (vec >= n * per_tok) return;
    const uint32_t t = vec / per_tok, h = vec % per_tok;
    const bool is_k = h >= heads;
    const uint32_t kh = h - heads;
    float *qrow = q + ((size_t)t * heads + h) * hd;
    const float *src = is_k ? k + ((size_t)t * kvh + kh) * hd : qrow;
    const float *nw = is_k ? k_norm : q_norm;
    constexpr int kMax = 8;  // head dims up to 256
    float x[kMax];
    float ss = 0.0f;
#pragma unroll
    for (int r = 0; r < kMax; ++r) {
        const uint32_t e = lane + 32u * r;
        x[r] = e < hd ? src[e] : 0.0f;
        ss = fmaf(x[r], x[r], ss);
    }
#pragma unroll
    for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
    const float inv = 1.0f / sqrtf(ss / (float)hd + eps);
#pragma unroll
    for (int r = 0; r < kMax; ++r) {
        const uint32_t e = lane + 32u * r;
        if (e < hd) x[r] = x[r] * inv * nw[e];
    }
    // Pairs (i, i + n_rot/2): with lane-strided elements the partner sits r_half registers away in the
    // same lane when n_rot/2 is a multiple of 32, otherwise it is fetched from another lane.
    const uint32_t half = n_rot / 2u, pos = pos0 + t;
    float y[kMax];
#pragma unroll
    for (int r = 0; r < kMax; ++r) y[r] = x[r];
#pragma unroll
    for (int r = 0; r < kMax; ++r) {
        const uint32_t e = lane + 32u * r;
        // partner element index and whether e is the first or the second member of its pair
        const bool first = e < half, second = e >= half && e < n_rot;
        const uint32_t pe = first ? e + half : e - half;
        float partner = 0.0f;
        // the partner lives at register (pe / 32) of lane (pe % 32); when half the rotated width is a
        // multiple of 32 (head sizes 64 and up, fully rotated) that is this lane: no shuffles
        if ((half & 31u) == 0u) {
#pragma unroll
            for (int rr = 0; rr < kMax; ++rr)
                if ((first || second) && (uint32_t)rr == (pe >> 5)) partner = x[rr];
        } else {
#pragma unroll
            for (int rr = 0; rr < kMax; ++rr) {
                const float cand = __shfl_sync(0xffffffffu, x[rr], (int)(pe & 31u));
                if ((first || second) && (uint32_t)rr == (pe >> 5)) partner = cand;
            }
        }
        if (first || second) {
            const uint32_t i = first ? e : e - half;
            float sn, cs;
            sincosf((float)pos * inv_freq[i], &sn, &cs);
            y[r] = first ? x[r] * cs - partner * sn : partner * sn + x[r] * cs;
        }
    }
    if (!is_k) {
#pragma unroll
        for (int r = 0; r < kMax; ++r) {
            const uint32_t e = lane + 32u * r;
            if (e < hd) qrow[e] = y[r];
        }
    } else {
        const float *vsrc = v + ((size_t)t * kvh + kh) * hd;
        const size_t dst = ((size_t)kh * cap + pos) * hd;
#pragma unroll
        for (int r = 0; r < kMax; ++r) {
            const uint32_t e = lane + 32u * r;
            if (e < hd) {
                kc[dst + e] = __float2half_rn(y[r]);
                vc[dst + e] = __float2half_rn(vsrc[e]);
            }
        }
    }
}

// ---- decode attention for many sequences on the tensor cores ---------------------------------
// The per-token core (per-head q/k RMS norm, RoPE, f16 KV store, windowed causal attention) for one
// row per sequence, throughput form: when tens of sequences decode together the step reads every
// sequence's K and V rows and is bandwidth-bound, which the latency-optimised kernel (scalar dot
// products, two threads per key) cannot feed.  Here one CTA of 4 warps serves ONE (sequence, KV head,
// split of `tiles` 64-key tiles): the G query heads of the group are the rows of a 16-row MMA tile,
// K/V tiles arrive by cp.async (double-buffered), warp w owns keys 16w..16w+15 of every tile with its
// own running (max, sum, output), the four are merged through shared memory, and the splits of a
// (sequence, KV head) by last arrival through `scratch` (no waiting).  Same mathematics as the other
// decode kernels, f16 Q and softmax weights, base-2 exponentials: tolerance-qualified.
//   scratch (per sequence): float part[kv_heads][nsplit][G][HD + 2] = (m, l, o[HD]); then, at the offset
//   the other decode kernels use, u32 count[kv_heads] (left at zero).
struct decode_mma_args {
    const float *q, *k, *v, *q_norm, *k_norm, *inv_freq;
    __half *kc, *vc;
    float *out, *scratch;
    const uint32_t *pos;
    uint32_t *status;
    uint32_t kv_heads, cap, window, tiles, count_off;  // count_off: floats from a sequence's scratch to its counters
    float eps, scale_log2e;
    size_t sq, sk, sv, so, scache, sscratch;  // element strides between sequences
};

template <int G, int HD>
__global__ void __launch_bounds__(kThreads) attention_decode_mma_kernel(const decode_mma_args a) {
    constexpr int PITCH = HD * 2, EPL = HD / 32;
    constexpr uint32_t kQBytes = 16 * PITCH, kTile = kBKV * PITCH, kStage = 2 * kTile;
    extern __shared__ __align__(128) unsigned char smem[];
    unsigned char *sQ = smem, *sKV = smem + kQBytes;
    __shared__ __align__(16) __half kh[HD];
    __shared__ __align__(16) __half vh[HD];
    __shared__ float wm[4][G], wl[4][G];
    __shared__ uint32_t s_last;
    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const int g = lane >> 2, t = lane & 3;
    const uint32_t kvh = blockIdx.x, split = blockIdx.y;
    const size_t sidx = blockIdx.z;
    const float *q = a.q + sidx * a.sq, *k = a.k + sidx * a.sk, *v = a.v + sidx * a.sv;
    __half *kc = a.kc + sidx * a.scache + (size_t)kvh * a.cap * HD, *vc = a.vc + sidx * a.scache + (size_t)kvh * a.cap * HD;
    float *out = a.out + sidx * a.so, *scratch = a.scratch + sidx * a.sscratch;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    asm volatile("griddepcontrol.launch_dependents;");
    const uint32_t pos = a.pos[sidx];
    if (pos >= a.cap) {
        if (tid == 0 && split == 0 && kvh == 0) atomicOr(a.status, 1u);
        return;
    }
    const uint32_t seq = pos + 1u, start = (a.window != 0u && seq > a.window) ? seq - a.window : 0u;
    const uint32_t first_tile = start / kBKV, last_tile = pos / kBKV;
    const uint32_t tile_lo = first_tile + split * a.tiles;
    if (tile_lo > last_tile) return;
    const uint32_t tile_hi = min(tile_lo + a.tiles - 1u, last_tile);
    const uint32_t nact = (last_tile - first_tile) / a.tiles + 1u;  // splits of this (sequence, KV head)
    const bool owns_new = tile_hi == last_tile;

    auto load_tile = [&](uint32_t tile, int stage) {
        unsigned char *sK = sKV + stage * kStage, *sV = sK + kTile;
        const uint32_t j0 = tile * kBKV;
        constexpr int CH = HD / 8;  // 16-byte chunks per row
        for (int i = tid; i < kBKV * CH; i += kThreads) {
            const uint32_t r = i / CH, c = i % CH;
            const uint32_t j = min(j0 + r, pos);  // rows past the position repeat its row (masked below)
            cp_async16(smem_u32(sK) + sw<PITCH>(r, c), kc + (size_t)j * HD + c * 8);
            cp_async16(smem_u32(sV) + sw<PITCH>(r, c), vc + (size_t)j * HD + c * 8);
        }
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    load_tile(tile_lo, 0);

    // ---- q_0..q_{G-1} (and k, v for the split that holds the position): RMS norm + RoPE, a warp each ----
    for (int i = tid; i < 16 * (HD / 8); i += kThreads) *(uint4 *)(sQ + i * 16) = make_uint4(0, 0, 0, 0);
    __syncthreads();
    for (int vec = warp; vec < G + (owns_new ? 1 : 0); vec += kThreads / 32) {
        const bool is_k = vec == G;
        const float *src = is_k ? k + (size_t)kvh * HD : q + ((size_t)kvh * G + vec) * HD;
        const float *nw = is_k ? a.k_norm : a.q_norm;
        float x[EPL];
        float ss = 0.0f;
#pragma unroll
        for (int r = 0; r < EPL; ++r) {
            x[r] = src[lane + 32 * r];
            ss = fmaf(x[r], x[r], ss);
        }
#pragma unroll
        for (int off = 16; off > 0; off >>= 1) ss += __shfl_xor_sync(0xffffffffu, ss, off);
        const float inv = 1.0f / sqrtf(ss / (float)HD + a.eps);
#pragma unroll
        for (int r = 0; r < EPL; ++r) x[r] = x[r] * inv * nw[lane + 32 * r];
        // full rotation: pair (i, i + HD/2), i = lane + 32 r, has both members in this lane
#pragma unroll
        for (int r = 0; r < EPL / 2; ++r) {
            float sn, cs;
            sincosf((float)pos * a.inv_freq[lane + 32 * r], &sn, &cs);
            const float a0 = x[r], b0 = x[r + EPL / 2];
            x[r] = a0 * cs - b0 * sn;
            x[r + EPL / 2] = a0 * sn + b0 * cs;
        }
        if (is_k) {
            const float *vsrc = v + (size_t)kvh * HD;
#pragma unroll
            for (int r = 0; r < EPL; ++r) {
                const uint32_t e = lane + 32 * r;
                const __half hk = __float2half_rn(x[r]), hv = __float2half_rn(vsrc[e]);
                kh[e] = hk;
                vh[e] = hv;
                kc[(size_t)pos * HD + e] = hk;
                vc[(size_t)pos * HD + e] = hv;
            }
        } else {
#pragma unroll
            for (int r = 0; r < EPL; ++r) {
                const uint32_t e = lane + 32 * r;
                *(__half *)(sQ + sw<PITCH>((uint32_t)vec, e >> 3) + (e & 7u) * 2u) = __float2half_rn(x[r]);
            }
        }
    }

    // This warp's running state over its 16 keys of every tile; rows g < G are the group's heads.
    float o[HD / 8][4];
#pragma unroll
    for (int i = 0; i < HD / 8; ++i) o[i][0] = o[i][1] = o[i][2] = o[i][3] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;
    const bool row_live = g < G;

    for (uint32_t tile = tile_lo; tile <= tile_hi; ++tile) {
        const int stage = (int)((tile - tile_lo) & 1u);
        if (tile < tile_hi) {
            load_tile(tile + 1, stage ^ 1);
            asm volatile("cp.async.wait_group 1;" ::: "memory");
        } else {
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
        __syncthreads();  // the tile has landed (and, first time round, Q and the new row are written)
        const uint32_t j0 = tile * kBKV;
        if (tile == last_tile) {  // the position's own row comes from this step, not from the cache
            const uint32_t r = pos - j0;
            unsigned char *sK = sKV + stage * kStage, *sV = sK + kTile;
            if (tid < HD / 8) *(uint4 *)(sK + sw<PITCH>(r, tid)) = *(const uint4 *)(kh + tid * 8);
            else if (tid < HD / 4) *(uint4 *)(sV + sw<PITCH>(r, tid - HD / 8)) = *(const uint4 *)(vh + (tid - HD / 8) * 8);
            __syncthreads();
        }
        const uint32_t sK = smem_u32(sKV + stage * kStage), sV = sK + kTile;
        // ---- S = Q K^T: 16 rows x this warp's 16 keys ----
        float s[2][4];
#pragma unroll
        for (int i = 0; i < 2; ++i) s[i][0] = s[i][1] = s[i][2] = s[i][3] = 0.0f;
#pragma unroll
        for (int kt = 0; kt < HD / 16; ++kt) {
            uint32_t a0, a1, a2, a3, b0, b1, b2, b3;
            const uint32_t m = lane >> 3;
            ldsm_x4(smem_u32(sQ) + sw<PITCH>((m & 1u) * 8 + (lane & 7), kt * 2 + (m >> 1)), a0, a1, a2, a3);
            ldsm_x4(sK + sw<PITCH>(warp * 16 + (m >> 1) * 8 + (lane & 7), kt * 2 + (m & 1u)), b0, b1, b2, b3);
            mma_f16(s[0], a0, a1, a2, a3, b0, b1);
            mma_f16(s[1], a0, a1, a2, a3, b2, b3);
        }
        // ---- mask, running maximum, weights (rows g only: rows g + 8 are padding) ----
        float mx = -INFINITY;
#pragma unroll
        for (int i = 0; i < 2; ++i)
#pragma unroll
            for (int e = 0; e < 2; ++e) {
                const uint32_t j = j0 + warp * 16 + i * 8 + 2 * t + e;
                const bool vis = row_live && j >= start && j <= pos;
                s[i][e] = vis ? s[i][e] * a.scale_log2e : -INFINITY;
                mx = fmaxf(mx, s[i][e]);
            }
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 1));
        mx = fmaxf(mx, __shfl_xor_sync(0xffffffffu, mx, 2));
        const float m_new = fmaxf(m_run, mx);
        const float m_use = m_new == -INFINITY ? 0.0f : m_new;
        const float alpha = exp2f(m_run - m_use);
        m_run = m_new;
        const float p00 = exp2f(s[0][0] - m_use), p01 = exp2f(s[0][1] - m_use);
        const float p10 = exp2f(s[1][0] - m_use), p11 = exp2f(s[1][1] - m_use);
        float rs = p00 + p01 + p10 + p11;
        rs += __shfl_xor_sync(0xffffffffu, rs, 1);
        rs += __shfl_xor_sync(0xffffffffu, rs, 2);
        l_run = l_run * alpha + rs;
        const uint32_t pa0 = pack_h2(p00, p01), pa2 = pack_h2(p10, p11);  // rows g: keys 0-7 / 8-15; rows g + 8: zero
#pragma unroll
        for (int i = 0; i < HD / 8; ++i) {
            o[i][0] *= alpha;
            o[i][1] *= alpha;
        }
        // ---- O += P V over this warp's 16 keys ----
#pragma unroll
        for (int dp = 0; dp < HD / 16; ++dp) {
            uint32_t b0, b1, b2, b3;
            const uint32_t m = lane >> 3;
            ldsm_x4_t(sV + sw<PITCH>(warp * 16 + (m & 1u) * 8 + (lane & 7), dp * 2 + (m >> 1)), b0, b1, b2, b3);
            mma_f16(o[2 * dp], pa0, 0u, pa2, 0u, b0, b1);
            mma_f16(o[2 * dp + 1], pa0, 0u, pa2, 0u, b2, b3);
        }
        __syncthreads();  // the stage is refilled by the next iteration's prefetch
    }

    // ---- the four warps' (m, l, o) -> this split's; the K/V stages are free now ----
    float *wo = (float *)sKV;  // [4][G][HD]
    if (row_live) {
        if (t == 0) {
            wm[warp][g] = m_run;
            wl[warp][g] = l_run;
        }
#pragma unroll
        for (int i = 0; i < HD / 8; ++i)
            *(float2 *)(wo + ((size_t)warp * G + g) * HD + i * 8 + 2 * t) = make_float2(o[i][0], o[i][1]);
    }
    __syncthreads();
    constexpr uint32_t stride = HD + 2;
    const uint32_t nsplit = gridDim.y;
    float *part = scratch + ((size_t)kvh * nsplit + split) * G * stride;
    const bool single = nact == 1u;
    for (uint32_t i = tid; i < G * HD; i += kThreads) {
        const uint32_t gg = i / HD, d = i % HD;
        float M = fmaxf(fmaxf(wm[0][gg], wm[1][gg]), fmaxf(wm[2][gg], wm[3][gg]));
        float L = 0.0f, O = 0.0f;
#pragma unroll
        for (int w = 0; w < 4; ++w) {
            const float f = exp2f(wm[w][gg] - M);  // a warp that saw no key: exp2(-inf) = 0
            L = fmaf(f, wl[w][gg], L);
            O = fmaf(f, wo[((size_t)w * G + gg) * HD + d], O);
        }
        if (single) {
            out[((size_t)kvh * G + gg) * HD + d] = O / L;
        } else {
            part[gg * stride + 2 + d] = O;
            if (d == 0) {
                part[gg * stride] = M;
                part[gg * stride + 1] = L;
            }
        }
    }
    if (single) return;
    __threadfence();
    __syncthreads();
    uint32_t *count = (uint32_t *)(scratch + a.count_off) + kvh;
    if (tid == 0) s_last = atomicAdd(count, 1u) == nact - 1u ? 1u : 0u;
    __syncthreads();
    if (!s_last) return;
    __threadfence();
    for (uint32_t i = tid; i < G * HD; i += kThreads) {
        const uint32_t gg = i / HD, d = i % HD;
        const float *base = scratch + (size_t)kvh * nsplit * G * stride + gg * stride;
        float M = -INFINITY, L = 0.0f, O = 0.0f;
        for (uint32_t s0 = 0; s0 < nact; s0 += 8) {
            float mb[8], lb[8], ob[8];
#pragma unroll
            for (int c = 0; c < 8; ++c) {
                const float *pb = base + (size_t)(s0 + c < nact ? s0 + c : nact - 1) * G * stride;
                mb[c] = __ldcg(pb);
                lb[c] = __ldcg(pb + 1);
                ob[c] = __ldcg(pb + 2 + d);
            }
            float mx = M;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                if (s0 + c < nact) mx = fmaxf(mx, mb[c]);
            const float al = exp2f(M - mx);
            L *= al;
            O *= al;
#pragma unroll
            for (int c = 0; c < 8; ++c)
                if (s0 + c < nact) {
                    const float wgt = exp2f(mb[c] - mx);
                    L = fmaf(wgt, lb[c], L);
                    O = fmaf(wgt, ob[c], O);
                }
            M = mx;
        }
        out[((size_t)kvh * G + gg) * HD + d] = O / L;
    }
    if (tid == 0) *count = 0u;  // ready for the next launch on this stream
}

template <int G, int HD>
cudaError_t launch_decode_mma(tm_cuda_ctx *ctx, const decode_mma_args &a, uint32_t n_seq) {
    constexpr uint32_t kBytes = 16 * HD * 2 + 2 * 2 * kBKV * HD * 2;
    static std::atomic<bool> attr_done[64] = {};
    const int device = ctx->device;
    if (device < 0 || device >= 64 || !attr_done[device].load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(attention_decode_mma_kernel<G, HD>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kBytes);
        if (e != cudaSuccess) return e;
        if (device >= 0 && device < 64) attr_done[device].store(true, std::memory_order_release);
    }
    const uint32_t n_tiles = (a.cap + kBKV - 1) / kBKV;
    const dim3 grid(a.kv_heads, (n_tiles + a.tiles - 1) / a.tiles, n_seq);
    return tm_launch_pdl(ctx, attention_decode_mma_kernel<G, HD>, grid, dim3(kThreads), kBytes, a);
}

template <int HD>
cudaError_t launch_attn(const attn_args &a, int device, cudaStream_t stream) {
    using C = attn_cfg<HD>;
    static std::atomic<bool> attr_done[64] = {};  // per device; contexts of a process share it
    if (device < 0 || device >= 64 || !attr_done[device].load(std::memory_order_acquire)) {
        const cudaError_t e = cudaFuncSetAttribute(attention_chunk_mma_kernel<HD>,
                                                   cudaFuncAttributeMaxDynamicSharedMemorySize, (int)C::kBytes);
        if (e != cudaSuccess) return e;
        if (device >= 0 && device < 64) attr_done[device].store(true, std::memory_order_release);
    }
    const dim3 grid((a.n + kBQ - 1) / kBQ, a.heads, HD / C::kDV);
    attention_chunk_mma_kernel<HD><<<grid, kThreads, C::kBytes, stream>>>(a);
    return cudaGetLastError();
}

}  // namespace

// Whether the tensor-core decode form serves this geometry.
bool tm_attention_decode_mma_ok(uint32_t heads, uint32_t kv_heads, uint32_t hd, uint32_t n_rot) {
    const uint32_t g = kv_heads ? heads / kv_heads : 0;
    return hd == 128 && n_rot == hd && (g == 1 || g == 2 || g == 4);
}

// One launch for n_seq sequences (pointers are sequence 0's; strides in elements between sequences).
cudaError_t tm_attention_decode_mma_launch(tm_cuda_ctx *ctx, const float *q, const float *k, const float *v,
                                           const float *qn, const float *kn, const float *inv_freq, void *kc, void *vc,
                                           float *out, float *scratch, const uint32_t *pos, uint32_t *status,
                                           uint32_t heads, uint32_t kv_heads, uint32_t hd, uint32_t cap, uint32_t window,
                                           float eps, float scale, uint32_t n_seq, size_t sq, size_t skv, size_t so,
                                           size_t scache, size_t sscratch, uint32_t count_off) {
    decode_mma_args a;
    a.q = q; a.k = k; a.v = v; a.q_norm = qn; a.k_norm = kn; a.inv_freq = inv_freq;
    a.kc = (__half *)kc; a.vc = (__half *)vc;
    a.out = out; a.scratch = scratch; a.pos = pos; a.status = status;
    a.kv_heads = kv_heads; a.cap = cap; a.window = window;
    a.count_off = count_off;
    a.eps = eps;
    a.scale_log2e = scale * 1.4426950408889634f;
    a.sq = sq; a.sk = a.sv = skv; a.so = so; a.scache = scache; a.sscratch = sscratch;
    // Keys per CTA: enough CTAs to fill the machine a few times over, as few splits as that allows.
    const uint32_t n_tiles = (cap + kBKV - 1) / kBKV;
    uint32_t tiles = 8;
    while (tiles > 1 && (uint64_t)n_seq * kv_heads * ((n_tiles + tiles - 1) / tiles) < 4ull * (uint64_t)ctx->sm_count) tiles >>= 1;
    a.tiles = tiles;
    (void)hd;
    switch (heads / kv_heads) {
        case 1: return launch_decode_mma<1, 128>(ctx, a, n_seq);
        case 2: return launch_decode_mma<2, 128>(ctx, a, n_seq);
        default: return launch_decode_mma<4, 128>(ctx, a, n_seq);
    }
}

extern "C" {

int tm_cuda_attention_chunk_mma_supported(uint32_t head_dim) {
    return head_dim == 32 || head_dim == 64 || head_dim == 128 || head_dim == 256;
}

int tm_cuda_qk_prep_chunk(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k, tm_cuda_buffer *v,
                          tm_cuda_buffer *q_norm, tm_cuda_buffer *k_norm, tm_cuda_buffer *inv_freq,
                          tm_cuda_buffer *k_cache, tm_cuda_buffer *v_cache, uint32_t heads, uint32_t kv_heads,
                          uint32_t head_dim, uint32_t n_rot, uint32_t pos0, uint32_t cap, uint32_t n, float eps,
                          char *err, size_t err_cap) {
    TM_ENTER();
    if (heads == 0 || kv_heads == 0 || head_dim == 0 || head_dim > 256 || n_rot == 0 || n_rot > head_dim ||
        n_rot % 2 != 0 || n == 0 || (size_t)pos0 + n > cap)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "q/k preparation: heads %u/%u, head_dim %u (<= 256), n_rot %u, rows %u..%u of capacity %u", heads,
                       kv_heads, head_dim, n_rot, pos0, pos0 + n, cap);
    const size_t plane = (size_t)kv_heads * cap * head_dim * 2;
    TM_CHECK_BUF(q, (size_t)n * heads * head_dim * 4, "q");
    TM_CHECK_BUF(k, (size_t)n * kv_heads * head_dim * 4, "k");
    TM_CHECK_BUF(v, (size_t)n * kv_heads * head_dim * 4, "v");
    TM_CHECK_BUF(q_norm, (size_t)head_dim * 4, "q norm");
    TM_CHECK_BUF(k_norm, (size_t)head_dim * 4, "k norm");
    TM_CHECK_BUF(inv_freq, (size_t)(n_rot / 2) * 4, "inv_freq");
    TM_CHECK_BUF(k_cache, plane, "K cache");
    TM_CHECK_BUF(v_cache, plane, "V cache");
    TM_OP_BEGIN("qk_prep_chunk");
    const uint32_t vecs = n * (heads + kv_heads);
    qk_prep_chunk_kernel<<<(vecs + 7) / 8, 256, 0, ctx->stream>>>(
        (float *)q->dev, (const float *)k->dev, (const float *)v->dev, (const float *)q_norm->dev,
        (const float *)k_norm->dev, (const float *)inv_freq->dev, (__half *)k_cache->dev, (__half *)v_cache->dev, heads,
        kv_heads, head_dim, n_rot, pos0, cap, n, eps);
    TM_OP_END(1);
}

int tm_cuda_attention_chunk_mma(tm_cuda_ctx *ctx, tm_cuda_buffer *q, tm_cuda_buffer *k_cache, tm_cuda_buffer *v_cache,
                                tm_cuda_buffer *out, uint32_t heads, uint32_t pos0, uint32_t cap, uint32_t head_dim,
                                uint32_t group, float scale, uint32_t n, uint32_t window, char *err, size_t err_cap) {
    TM_ENTER();
    if (!tm_cuda_attention_chunk_mma_supported(head_dim) || heads == 0 || group == 0 || heads % group != 0 || n == 0 ||
        cap == 0 || (size_t)pos0 + n > cap)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS,
                       "tensor-core chunk attention: heads %u, group %u, head_dim %u (32, 64, 128 or 256), rows "
                       "%u..%u of capacity %u", heads, group, head_dim, pos0, pos0 + n, cap);
    const uint32_t kv_heads = heads / group;
    const size_t plane = (size_t)kv_heads * cap * head_dim * 2;
    TM_CHECK_BUF(q, (size_t)n * heads * head_dim * 4, "q");
    TM_CHECK_BUF(out, (size_t)n * heads * head_dim * 4, "attention output");
    TM_CHECK_BUF(k_cache, plane, "K cache");
    TM_CHECK_BUF(v_cache, plane, "V cache");
    if (((size_t)q->dev | (size_t)out->dev | (size_t)k_cache->dev | (size_t)v_cache->dev) & 15u)
        return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "tensor-core chunk attention needs 16-byte aligned buffers");
    attn_args a;
    a.q = (const float *)q->dev;
    a.kc = (const __half *)k_cache->dev;
    a.vc = (const __half *)v_cache->dev;
    a.out = (float *)out->dev;
    a.heads = heads;
    a.group = group;
    a.pos0 = pos0;
    a.cap = cap;
    a.n = n;
    a.window = window;
    a.scale_log2e = scale * 1.4426950408889634f;
    TM_OP_BEGIN("attention_chunk_mma");
    cudaError_t e = head_dim == 32    ? launch_attn<32>(a, ctx->device, ctx->stream)
                    : head_dim == 64  ? launch_attn<64>(a, ctx->device, ctx->stream)
                    : head_dim == 128 ? launch_attn<128>(a, ctx->device, ctx->stream)
                                      : launch_attn<256>(a, ctx->device, ctx->stream);
    TM_CUDA_TRY(e);
    TM_OP_END(1);
}

}  // extern "C"
