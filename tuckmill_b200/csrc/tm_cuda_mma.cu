// Prefill GEMM on the 5th-generation tensor cores (tcgen05 + tensor memory).
//
// Contract (the reference's matrix-unit GEMM, native/metal/kernels.metal:503-635
// and native/metal/tm_metal.h:168-189): Y[b, :] = W X[b, :] for b < batch, X at
// f32 offset x_off, Y at y_off, tolerance-qualified.  The reference multiplies
// f32 operands on 8x8 SIMD-group tiles; this kernel follows the declared f16
// operand profile instead: x and d*q are rounded to binary16 (each once, to
// nearest even), products accumulate in f32 in tensor memory.
//
// One CTA computes a 128 (weight rows) x BN (tokens) tile of Y^T:
//   warps 0-3  producers: each thread owns one weight row of the tile, loads 64
//              int8 quants + 2 scales per K block straight from the packed
//              planes, converts to f16 (byte permute into 1024+u, subtract
//              1152, multiply by d) and writes the row into the 128-byte
//              swizzled K-major layout the MMA reads; later the epilogue
//   warp 4     one thread issues the TMA loads of the token tile (f16 copy of X)
//   warp 5     allocates tensor memory; one thread issues tcgen05.mma
// Stages are handed over with mbarriers; every wait is bounded and raises an
// abort flag instead of spinning forever.
#include <cuda.h>

#include "tm_cuda_internal.cuh"

namespace {

constexpr int kBM = 128;        // weight rows per tile (UMMA M)
constexpr int kBK = 64;         // K per stage: 64 f16 = one 128-byte swizzle row
constexpr int kStages = 4;
constexpr int kMmaThreads = 192;
constexpr uint32_t kSpinLimit = 1u << 20;  // a healthy wait is microseconds; this is ~seconds

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

__device__ __forceinline__ void umma_f16(uint32_t d_tmem, uint64_t a_desc, uint64_t b_desc, uint32_t idesc,
                                         uint32_t accumulate) {
    asm volatile(
        "{\n .reg .pred p;\n setp.ne.b32 p, %4, 0;\n"
        " tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n}\n" ::"r"(d_tmem),
        "l"(a_desc), "l"(b_desc), "r"(idesc), "r"(accumulate)
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
__device__ __forceinline__ int4 dequant8(uint32_t w0, uint32_t w1, __half2 d2) {
    const __half2 bias = __half2half2(__ushort_as_half((unsigned short)0x6480));  // 1152.0
    uint32_t out[4];
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
    return make_int4((int)out[0], (int)out[1], (int)out[2], (int)out[3]);
}

struct mma_args {
    const signed char *q;  // [rows][cols]
    const __half *d;       // [rows][cols/32]
    float *y;              // Y[t * rows + r]
    uint32_t rows, cols, batch;
    uint32_t *abort_flag;  // set when a bounded wait gave up
};

template <int BN>
__global__ void __launch_bounds__(kMmaThreads, 1) q8_gemm_mma_kernel(const __grid_constant__ CUtensorMap xmap,
                                                                     const mma_args a) {
    extern __shared__ __align__(1024) unsigned char smem_raw[];
    // 1024-byte aligned stage buffers (swizzle atoms), then the barriers.
    unsigned char *smem = (unsigned char *)(((uintptr_t)smem_raw + 1023) & ~(uintptr_t)1023);
    constexpr uint32_t kABytes = kBM * kBK * 2, kBBytes = BN * kBK * 2;
    unsigned char *sA = smem, *sB = smem + kStages * kABytes;
    uint64_t *full_a = (uint64_t *)(sB + kStages * kBBytes);
    uint64_t *full_b = full_a + kStages, *empty = full_b + kStages, *accum = empty + kStages;
    uint32_t *tmem_slot = (uint32_t *)(accum + 1);
    volatile uint32_t *abort_s = tmem_slot + 1;

    const int tid = threadIdx.x, warp = tid >> 5, lane = tid & 31;
    const uint32_t row0 = blockIdx.x * kBM, tok0 = blockIdx.y * BN;
    const uint32_t nkb = (a.cols + kBK - 1) / kBK, nb = a.cols / 32u;

    if (tid == 0) {
        for (int s = 0; s < kStages; ++s) {
            mbar_init(&full_a[s], 4);  // one arrival per producer warp
            mbar_init(&full_b[s], 1);  // the TMA thread's expect_tx arrival
            mbar_init(&empty[s], 1);   // tcgen05.commit
        }
        mbar_init(accum, 1);
        *abort_s = 0u;
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 5) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(smem_u32(tmem_slot)),
                     "r"((uint32_t)BN)
                     : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    const uint32_t tmem_base = *tmem_slot;

    if (warp < 4) {
        // ---------------- producers: dequantise one weight row per thread ----------------
        const uint32_t r = min(row0 + (uint32_t)tid, a.rows - 1u);  // rows past the end repeat the last (masked later)
        const signed char *qrow = a.q + (size_t)r * a.cols;
        const __half *drow = a.d + (size_t)r * nb;
        int4 raw[4];
        __half sc[2];
        auto fetch = [&](uint32_t kb) {
            const uint32_t k0 = kb * kBK;
#pragma unroll
            for (int c = 0; c < 4; ++c)
                raw[c] = k0 + c * 16 < a.cols ? *(const int4 *)(qrow + k0 + c * 16) : make_int4(0, 0, 0, 0);
            sc[0] = k0 < a.cols ? drow[k0 / 32] : __ushort_as_half((unsigned short)0);
            sc[1] = k0 + 32 < a.cols ? drow[k0 / 32 + 1] : __ushort_as_half((unsigned short)0);
        };
        fetch(0);
        bool ok = true;
        for (uint32_t kb = 0; kb < nkb && ok; ++kb) {
            const uint32_t s = kb % kStages, it = kb / kStages;
            if (it > 0) ok = mbar_wait(&empty[s], (it - 1) & 1, abort_s);
            if (!ok) break;
            unsigned char *rowp = sA + s * kABytes + (uint32_t)tid * 128u;
#pragma unroll
            for (int c = 0; c < 8; ++c) {  // chunk c = k 8c..8c+7 of this K block
                const int4 w = raw[c >> 1];
                const uint32_t w0 = (c & 1) ? (uint32_t)w.z : (uint32_t)w.x, w1 = (c & 1) ? (uint32_t)w.w : (uint32_t)w.y;
                const int4 v = dequant8(w0, w1, __half2half2(sc[c >> 2]));
                *(int4 *)(rowp + ((c ^ (tid & 7)) << 4)) = v;
            }
            if (kb + 1 < nkb) fetch(kb + 1);  // next block's bytes travel while the MMA consumes this one
            asm volatile("fence.proxy.async.shared::cta;" ::: "memory");  // generic writes -> async proxy (UMMA)
            __syncwarp();
            if (lane == 0) mbar_arrive(&full_a[s]);
        }
        // ---------------- epilogue: TMEM -> registers -> Y ----------------
        if (ok) ok = mbar_wait(accum, 0, abort_s);
        ok = __all_sync(0xffffffffu, ok);  // the tensor-memory loads below are warp-collective
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        if (ok) {
            const uint32_t rr = row0 + (uint32_t)tid;
#pragma unroll 1
            for (int c0 = 0; c0 < BN; c0 += 32) {
                uint32_t v[32];
                const uint32_t taddr = tmem_base + ((uint32_t)(warp * 32) << 16) + (uint32_t)c0;
                asm volatile(
                    "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                    "{%0,%1,%2,%3,%4,%5,%6,%7,%8,%9,%10,%11,%12,%13,%14,%15,%16,%17,%18,%19,%20,%21,%22,%23,%24,%25,"
                    "%26,%27,%28,%29,%30,%31}, [%32];"
                    : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                      "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]),
                      "=r"(v[15]), "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]),
                      "=r"(v[22]), "=r"(v[23]), "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]),
                      "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                    : "r"(taddr)
                    : "memory");
                asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
                if (rr < a.rows) {
#pragma unroll
                    for (int j = 0; j < 32; ++j) {
                        const uint32_t t = tok0 + (uint32_t)(c0 + j);
                        if (t < a.batch) a.y[(size_t)t * a.rows + rr] = __uint_as_float(v[j]);
                    }
                }
            }
        }
    } else if (warp == 4) {
        // ---------------- TMA producer of the token tile ----------------
        if (lane == 0) {
            bool ok = true;
            for (uint32_t kb = 0; kb < nkb && ok; ++kb) {
                const uint32_t s = kb % kStages, it = kb / kStages;
                if (it > 0) ok = mbar_wait(&empty[s], (it - 1) & 1, abort_s);
                if (!ok) break;
                mbar_expect_tx(&full_b[s], kBBytes);
                tma_load_2d(sB + s * kBBytes, &xmap, (int)(kb * kBK), (int)tok0, &full_b[s]);
            }
        }
    } else {
        // ---------------- MMA issuer ----------------
        if (lane == 0) {
            constexpr uint32_t idesc = umma_idesc(kBM, BN);
            bool ok = true;
            for (uint32_t kb = 0; kb < nkb && ok; ++kb) {
                const uint32_t s = kb % kStages, it = kb / kStages;
                ok = mbar_wait(&full_a[s], it & 1, abort_s) && mbar_wait(&full_b[s], it & 1, abort_s);
                if (!ok) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
                const uint64_t da = umma_desc(smem_u32(sA + s * kABytes)), db = umma_desc(smem_u32(sB + s * kBBytes));
#pragma unroll
                for (uint32_t k = 0; k < kBK / 16; ++k)  // 16 f16 = 32 bytes = 2 descriptor units per step
                    umma_f16(tmem_base, da + 2 * k, db + 2 * k, idesc, (kb | k) != 0 ? 1u : 0u);
                umma_commit(&empty[s]);  // frees the stage once these MMAs have read it
            }
            if (ok) umma_commit(accum);  // fires when every MMA above has completed
        }
    }
    // ---------------- teardown: everyone meets, tensor memory goes back ----------------
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (tid == 0 && *abort_s) atomicOr(a.abort_flag, 1u);
    if (warp == 5) {
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "r"((uint32_t)BN)
                     : "memory");
    }
}

// f32 -> f16 copy of the activations (round to nearest even), the TMA source.
__global__ void x_to_f16_kernel(const float *x, __half *out, size_t n) {
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
size_t mma_smem_bytes() {
    return 1024 + (size_t)kStages * (kBM * kBK * 2 + BN * kBK * 2) + (3 * kStages + 1) * 8 + 16;
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

size_t tm_cuda_mma_workspace_bytes(uint32_t cols, uint32_t batch) { return (size_t)cols * batch * 2; }

int tm_cuda_q8_0_gemm_mma(tm_cuda_ctx *ctx, tm_cuda_buffer *w, tm_cuda_buffer *x, tm_cuda_buffer *y, uint32_t rows,
                          uint32_t cols, uint32_t batch, uint32_t x_off, uint32_t y_off, char *err, size_t err_cap) {
    if (batch >= 1 && batch < 9) {
        // A handful of tokens is HBM-bound: the exact integer-tensor-core path serves it (and is tighter).
        return tm_cuda_q8_0_gemm(ctx, w, x, y, rows, cols, batch, x_off, y_off, err, err_cap);
    }
    {
        const size_t need = tm_cuda_mma_workspace_bytes(cols, batch);
        bool small;
        {
            if (!ctx) return tm_fail(err, err_cap, TM_CUDA_ERR_UNSUPPORTED, "null context");
            std::lock_guard<std::mutex> lock(ctx->mu);
            small = ctx->mma_scratch_bytes < need;
        }
        if (small) {
            int rc = tm_cuda_mma_workspace_reserve(ctx, need, err, err_cap);
            if (rc != TM_CUDA_OK) return rc;
        }
    }
    TM_ENTER();
    int rc = tm_check_packed(ctx, w, rows, cols, err, err_cap);
    if (rc != TM_CUDA_OK) return rc;
    if (batch == 0 || batch > TM_CUDA_GEMM_MMA_MAX_BATCH)
        return tm_fail(err, err_cap, TM_CUDA_ERR_BOUNDS, "batch %u outside 1..%u", batch, TM_CUDA_GEMM_MMA_MAX_BATCH);
    TM_CHECK_BUF(x, ((size_t)x_off + (size_t)batch * cols) * 4, "activation");
    TM_CHECK_BUF(y, ((size_t)y_off + (size_t)batch * rows) * 4, "output");
    encode_tiled_fn encode = get_encode_tiled();
    if (!encode)
        return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "the driver does not export cuTensorMapEncodeTiled");
    __half *xh = (__half *)ctx->mma_scratch;
    uint32_t *abort_flag = (uint32_t *)(ctx->mma_scratch + tm_round_up(ctx->mma_scratch_bytes, 256));
    const int bn = batch > 128 ? 256 : 128;
    CUtensorMap map;
    const cuuint64_t gdim[2] = {cols, batch};
    const cuuint64_t gstride[1] = {(cuuint64_t)cols * 2};
    const cuuint32_t box[2] = {(cuuint32_t)kBK, (cuuint32_t)bn};
    const cuuint32_t estr[2] = {1, 1};
    const CUresult cr = encode(&map, CU_TENSOR_MAP_DATA_TYPE_FLOAT16, 2, (void *)xh, gdim, gstride, box, estr,
                               CU_TENSOR_MAP_INTERLEAVE_NONE, CU_TENSOR_MAP_SWIZZLE_128B,
                               CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
    if (cr != CUDA_SUCCESS)
        return tm_fail(err, err_cap, TM_CUDA_ERR_INTERNAL, "cuTensorMapEncodeTiled failed (%d)", (int)cr);
    mma_args a;
    a.q = (const signed char *)w->qp;
    a.d = (const __half *)w->dp;
    a.y = (float *)y->dev + y_off;
    a.rows = rows;
    a.cols = cols;
    a.batch = batch;
    a.abort_flag = abort_flag;
    TM_OP_BEGIN("q8_0_gemm_mma");
    const size_t n = (size_t)batch * cols;
    const int cgrid = (int)((n / 4 + 255) / 256 > 148 * 8 ? 148 * 8 : (n / 4 + 255) / 256);
    x_to_f16_kernel<<<cgrid < 1 ? 1 : cgrid, 256, 0, ctx->stream>>>((const float *)x->dev + x_off, xh, n);
    const dim3 grid((rows + kBM - 1) / kBM, (batch + bn - 1) / bn);
    static bool attr_done[2][16] = {};
    const int dev = ctx->device < 16 ? ctx->device : 0;
    if (bn == 256) {
        if (!attr_done[1][dev]) {
            TM_CUDA_TRY(cudaFuncSetAttribute(q8_gemm_mma_kernel<256>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)mma_smem_bytes<256>()));
            attr_done[1][dev] = true;
        }
        q8_gemm_mma_kernel<256><<<grid, kMmaThreads, mma_smem_bytes<256>(), ctx->stream>>>(map, a);
    } else {
        if (!attr_done[0][dev]) {
            TM_CUDA_TRY(cudaFuncSetAttribute(q8_gemm_mma_kernel<128>, cudaFuncAttributeMaxDynamicSharedMemorySize,
                                             (int)mma_smem_bytes<128>()));
            attr_done[0][dev] = true;
        }
        q8_gemm_mma_kernel<128><<<grid, kMmaThreads, mma_smem_bytes<128>(), ctx->stream>>>(map, a);
    }
    TM_OP_END(2);
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
