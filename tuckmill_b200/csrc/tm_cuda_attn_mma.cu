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
