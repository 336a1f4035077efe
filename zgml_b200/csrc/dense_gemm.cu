// Dense prefill matmul for the sequence-model LINEAR op on the 5th-generation tensor cores:
//   dst[M, N] = bf16(src)[M, K] * W[N, K]^T (+ bias), W stored bfloat16 row-major (the checkpoint's [out, in]).
//
//   * tcgen05.mma.cta_group::1.kind::f16 on BF16 operands, one 128 x 128 fp32 accumulator per CTA in TMEM, issued by one
//     thread; K advances 64 (one 128-byte swizzle row) per pipeline stage.
//   * BOTH operands arrive by TMA (cp.async.bulk.tensor.2d, 128B swizzle) straight into the canonical K-major layout: the
//     weight matrix as it lies in the arena (out-of-range rows / k are zero-filled by the copy engine), the activations
//     from a bf16 scratch that a small conversion kernel fills (one rounding per activation; accumulation stays fp32).
//   * 6-stage mbarrier ring (32 KB per stage): TMA warp -> MMA warp -> (tcgen05.commit) -> stage free.  Four epilogue warps
//     read the accumulator (tcgen05.ld 32x32b), transpose 32 x 32 blocks through the idle stage memory, add the bias and
//     write 128-byte row segments.
//   * Every wait is bounded: a barrier that does not flip within ~1 s of polling raises a sticky device flag
//     (zg_dense_gemm_timeouts) and the CTA drains — its roles all give up the same way — frees its TMEM and returns.
//
// Used when the session keeps bfloat16 weights and M > 8 (decode rows stream the weights through the row kernels of
// seqops.cu); float32 sessions keep the exact SIMT tile.
#include "zg_internal.cuh"

#include <cuda.h>
#include <cuda_bf16.h>

namespace {

constexpr uint32_t BM = 128, BN = 128, BK = 64;
constexpr uint32_t kTileA = BM * BK * 2, kTileB = BN * BK * 2, kStage = kTileA + kTileB;
constexpr uint32_t kStages = 6;
constexpr uint32_t kThreads = 192;   // warp 0: TMA, warp 1: MMA + TMEM, warps 2-5: epilogue
constexpr uint32_t kTmemCols = 128;
constexpr uint32_t kSmem = kStages * kStage + 1024 + 256;
constexpr uint32_t kSpinLimit = 1u << 22;

__device__ unsigned int g_timeouts = 0;

__device__ __forceinline__ uint32_t smem_u32(const void* p) { return (uint32_t)__cvta_generic_to_shared(p); }
__device__ __forceinline__ void mbar_init(uint32_t bar, uint32_t count) {
    asm volatile("mbarrier.init.shared::cta.b64 [%0], %1;" ::"r"(bar), "r"(count) : "memory");
}
__device__ __forceinline__ void mbar_expect_tx(uint32_t bar, uint32_t bytes) {
    asm volatile("mbarrier.arrive.expect_tx.shared::cta.b64 _, [%0], %1;" ::"r"(bar), "r"(bytes) : "memory");
}
// false: gave up (the flag is raised; the caller stops issuing work and falls through to the common exit)
__device__ __forceinline__ bool mbar_wait(uint32_t bar, uint32_t parity) {
    for (uint32_t i = 0; i < kSpinLimit; i++) {
        uint32_t ok;
        asm volatile(
            "{\n\t.reg .pred p;\n\t"
            "mbarrier.try_wait.parity.shared::cta.b64 p, [%1], %2;\n\t"
            "selp.u32 %0, 1, 0, p;\n\t}" : "=r"(ok) : "r"(bar), "r"(parity) : "memory");
        if (ok) return true;
    }
    atomicAdd(&g_timeouts, 1u);
    return false;
}
__device__ __forceinline__ void tma_load_2d(uint32_t dst, const CUtensorMap* map, uint32_t c0, uint32_t c1, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.2d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3}], [%4];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(bar) : "memory");
}
__device__ __forceinline__ void tma_load_3d(uint32_t dst, const CUtensorMap* map, uint32_t c0, uint32_t c1, uint32_t c2, uint32_t bar) {
    asm volatile("cp.async.bulk.tensor.3d.shared::cluster.global.mbarrier::complete_tx::bytes [%0], [%1, {%2, %3, %4}], [%5];"
                 ::"r"(dst), "l"(map), "r"(c0), "r"(c1), "r"(c2), "r"(bar) : "memory");
}
// K-major, 128-byte swizzle, 8-row groups 1024 B apart
__device__ __forceinline__ uint64_t make_desc(uint32_t smem_addr) {
    uint64_t d = 0;
    d |= (uint64_t)((smem_addr & 0x3FFFF) >> 4);
    d |= (uint64_t)1 << 16;
    d |= (uint64_t)(1024 >> 4) << 32;
    d |= (uint64_t)1 << 46;
    d |= (uint64_t)2 << 61;
    return d;
}

// f32 rows -> dense bf16 [Mp][Kp] (zero padding), two k per thread
// (ctl: the rows are those of a per-sequence state buffer, `slot_stride` elements per slot; the slot is the control word's)
__global__ void k_to_bf16(const float* __restrict__ x, uint32_t x_rs, uint32_t* __restrict__ out, uint32_t kp2, uint32_t M, uint32_t K, const float* __restrict__ ctl,
                          uint32_t slot_stride) {
    if (ctl) x += (size_t)reinterpret_cast<const int*>(ctl)[ZG_CTL_SLOT] * slot_stride;
    const uint32_t m = blockIdx.y;
    for (uint32_t k2 = blockIdx.x * blockDim.x + threadIdx.x; k2 < kp2; k2 += gridDim.x * blockDim.x) {
        const uint32_t k = 2 * k2;
        const float a = (m < M && k < K) ? x[(size_t)m * x_rs + k] : 0.0f;
        const float b = (m < M && k + 1 < K) ? x[(size_t)m * x_rs + k + 1] : 0.0f;
        uint32_t r;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(r) : "f"(b), "f"(a));
        out[(size_t)m * kp2 + k2] = r;
    }
}

// the epilogue's activation (the kinds of the ACTIVATION op, shifted by one: 0 is none)
__device__ __forceinline__ float gemm_act(float z, uint32_t act, float p) {
    switch (act) {
        case 5: return p * tanhf(z / p);
        case 0: return z;
        case 1: { const float r = fmaxf(z, 0.0f); return r * r; }
        case 2: return z / (1.0f + expf(-z));
        case 3: return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * fmaf(0.044715f * z * z, z, z)));
        default: return fmaxf(z, 0.0f);
    }
}
struct GemmParams {
    float* out;
    const __nv_bfloat16* bias;
    uint32_t M, N, K, out_rs, out_vec4;
    uint32_t act;            // applied after the bias: 0 none, 1 relu^2, 2 silu, 3 gelu (tanh form), 4 relu, 5 smooth cap act_p * tanh(z / act_p)
    float act_p;
    const int* tile_group;   // GROUPED: weight matrix (third TMA coordinate) of every 128-row tile, -1: tile unused
};

// GROUPED: the rows are sorted by weight matrix (expert) in whole 128-row tiles; tile t multiplies with matrix tile_group[t]
// of the stacked [groups][N][K] weight tensor.
template <bool GROUPED, bool ACT>       // ACT: the epilogue applies p.act (its own instantiation: the plain epilogue stays as it was)
__global__ void __launch_bounds__(kThreads, 1)
dense_gemm_kernel(const __grid_constant__ CUtensorMap tmap_a, const __grid_constant__ CUtensorMap tmap_b, const GemmParams p) {
    int group = 0;
    if (GROUPED) {
        group = p.tile_group[blockIdx.y];
        if (group < 0) return;   // uniform over the CTA, before any barrier or TMEM allocation
    }
    extern __shared__ uint8_t dsm_raw[];
    const uint32_t base = (smem_u32(dsm_raw) + 1023u) & ~1023u;
    const uint32_t bars = base + kStages * kStage;
    const uint32_t full = bars, empty = bars + 8 * kStages, tmem_full = bars + 16 * kStages, tmem_slot = tmem_full + 8;
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t tile_n = blockIdx.x, tile_m = blockIdx.y;
    const uint32_t n_k = (p.K + BK - 1) / BK;

    if (threadIdx.x == 0) {
        for (uint32_t s = 0; s < kStages; s++) { mbar_init(full + 8 * s, 1); mbar_init(empty + 8 * s, 1); }
        mbar_init(tmem_full, 1);
        asm volatile("fence.mbarrier_init.release.cluster;" ::: "memory");
    }
    if (warp == 1) {
        asm volatile("tcgen05.alloc.cta_group::1.sync.aligned.shared::cta.b32 [%0], %1;" ::"r"(tmem_slot), "n"(kTmemCols) : "memory");
        asm volatile("tcgen05.relinquish_alloc_permit.cta_group::1.sync.aligned;" ::: "memory");
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
    uint32_t tmem_base;
    asm volatile("ld.shared.u32 %0, [%1];" : "=r"(tmem_base) : "r"(tmem_slot));

    if (warp == 0) {
        if (lane == 0) {
            for (uint32_t kt = 0; kt < n_k; kt++) {
                const uint32_t s = kt % kStages, ph = (kt / kStages) & 1;
                if (!mbar_wait(empty + 8 * s, ph ^ 1)) break;
                mbar_expect_tx(full + 8 * s, kStage);
                tma_load_2d(base + s * kStage, &tmap_a, kt * BK, tile_m * BM, full + 8 * s);
                if (GROUPED) tma_load_3d(base + s * kStage + kTileA, &tmap_b, kt * BK, tile_n * BN, (uint32_t)group, full + 8 * s);
                else tma_load_2d(base + s * kStage + kTileA, &tmap_b, kt * BK, tile_n * BN, full + 8 * s);
            }
        }
    } else if (warp == 1) {
        // instruction descriptor (kind::f16): D = F32, A = B = BF16, both K-major, N = BN, M = 128
        constexpr uint32_t idesc = (1u << 4) | (1u << 7) | (1u << 10) | ((BN >> 3) << 17) | ((128u >> 4) << 24);
        if (lane == 0) {
            for (uint32_t kt = 0; kt < n_k; kt++) {
                const uint32_t s = kt % kStages, ph = (kt / kStages) & 1;
                if (!mbar_wait(full + 8 * s, ph)) break;
                asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
#pragma unroll
                for (uint32_t k = 0; k < BK / 16; k++) {
                    const uint64_t da = make_desc(base + s * kStage + k * 32), db = make_desc(base + s * kStage + kTileA + k * 32);
                    const uint32_t accumulate = (kt | k) ? 1u : 0u;
                    asm volatile(
                        "{\n\t.reg .pred p;\n\t"
                        "setp.ne.b32 p, %4, 0;\n\t"
                        "tcgen05.mma.cta_group::1.kind::f16 [%0], %1, %2, %3, p;\n\t}"
                        ::"r"(tmem_base), "l"(da), "l"(db), "r"(idesc), "r"(accumulate) : "memory");
                }
                asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(empty + 8 * s) : "memory");
                if (kt + 1 == n_k)
                    asm volatile("tcgen05.commit.cta_group::1.mbarrier::arrive::one.shared::cluster.b64 [%0];" ::"r"(tmem_full) : "memory");
            }
        }
        __syncwarp();
    } else {
        // ── epilogue: warp w may touch TMEM lanes 32 (w % 4) .. + 31 ──
        const uint32_t ew = warp - 2, quarter = warp & 3;
        const bool ok = mbar_wait(tmem_full, 0);
        asm volatile("tcgen05.fence::after_thread_sync;" ::: "memory");
        const uint32_t m_base = tile_m * BM + quarter * 32;
        uint4* tb = reinterpret_cast<uint4*>(dsm_raw + (base - smem_u32(dsm_raw)) + ew * (32 * 36 * 4));   // the stages are idle now
#pragma unroll 1
        for (uint32_t c0 = 0; ok && c0 < BN; c0 += 32) {
            uint32_t v[32];
            const uint32_t taddr = tmem_base + ((quarter * 32) << 16) + c0;
            asm volatile(
                "tcgen05.ld.sync.aligned.32x32b.x32.b32 "
                "{%0, %1, %2, %3, %4, %5, %6, %7, %8, %9, %10, %11, %12, %13, %14, %15, "
                "%16, %17, %18, %19, %20, %21, %22, %23, %24, %25, %26, %27, %28, %29, %30, %31}, [%32];"
                : "=r"(v[0]), "=r"(v[1]), "=r"(v[2]), "=r"(v[3]), "=r"(v[4]), "=r"(v[5]), "=r"(v[6]), "=r"(v[7]),
                  "=r"(v[8]), "=r"(v[9]), "=r"(v[10]), "=r"(v[11]), "=r"(v[12]), "=r"(v[13]), "=r"(v[14]), "=r"(v[15]),
                  "=r"(v[16]), "=r"(v[17]), "=r"(v[18]), "=r"(v[19]), "=r"(v[20]), "=r"(v[21]), "=r"(v[22]), "=r"(v[23]),
                  "=r"(v[24]), "=r"(v[25]), "=r"(v[26]), "=r"(v[27]), "=r"(v[28]), "=r"(v[29]), "=r"(v[30]), "=r"(v[31])
                : "r"(taddr));
            asm volatile("tcgen05.wait::ld.sync.aligned;" ::: "memory");
#pragma unroll
            for (int i = 0; i < 8; i++) tb[lane * 9 + i] = make_uint4(v[4 * i], v[4 * i + 1], v[4 * i + 2], v[4 * i + 3]);
            __syncwarp();
            const uint32_t n0 = tile_n * BN + c0;
            if (n0 < p.N) {
                if (p.out_vec4 && n0 + 32 <= p.N) {
                    const uint32_t nn = n0 + 4 * (lane & 7);
                    float b[4] = {0.0f, 0.0f, 0.0f, 0.0f};
                    if (p.bias) for (int j = 0; j < 4; j++) b[j] = __bfloat162float(p.bias[nn + j]);
#pragma unroll
                    for (int it = 0; it < 8; it++) {
                        const uint32_t rr = it * 4 + (lane >> 3), mm = m_base + rr;
                        const uint4 o = tb[rr * 9 + (lane & 7)];
                        const float4 f = make_float4((ACT ? gemm_act(__uint_as_float(o.x) + b[0], p.act, p.act_p) : __uint_as_float(o.x) + b[0]), (ACT ? gemm_act(__uint_as_float(o.y) + b[1], p.act, p.act_p) : __uint_as_float(o.y) + b[1]), (ACT ? gemm_act(__uint_as_float(o.z) + b[2], p.act, p.act_p) : __uint_as_float(o.z) + b[2]),
                                                     (ACT ? gemm_act(__uint_as_float(o.w) + b[3], p.act, p.act_p) : __uint_as_float(o.w) + b[3]));
                        if (mm < p.M) *reinterpret_cast<float4*>(p.out + (size_t)mm * p.out_rs + nn) = f;
                    }
                } else if (n0 + lane < p.N) {
                    const uint32_t* tw = reinterpret_cast<const uint32_t*>(tb);
                    const float b = p.bias ? __bfloat162float(p.bias[n0 + lane]) : 0.0f;
                    for (int rr = 0; rr < 32; rr++)
                        if (m_base + rr < p.M) p.out[(size_t)(m_base + rr) * p.out_rs + n0 + lane] = (ACT ? gemm_act(__uint_as_float(tw[rr * 36 + lane]) + b, p.act, p.act_p) : __uint_as_float(tw[rr * 36 + lane]) + b);
                }
            }
            __syncwarp();
        }
    }
    asm volatile("tcgen05.fence::before_thread_sync;" ::: "memory");
    __syncthreads();
    if (warp == 1) asm volatile("tcgen05.dealloc.cta_group::1.sync.aligned.b32 %0, %1;" ::"r"(tmem_base), "n"(kTmemCols) : "memory");
}

typedef CUresult (*EncodeTiledFn)(CUtensorMap*, CUtensorMapDataType, cuuint32_t, void*, const cuuint64_t*, const cuuint64_t*,
                                  const cuuint32_t*, const cuuint32_t*, CUtensorMapInterleave, CUtensorMapSwizzle,
                                  CUtensorMapL2promotion, CUtensorMapFloatOOBfill);
EncodeTiledFn g_encode = nullptr;
bool g_attr_set = false;

bool prepare() {
    if (!g_encode) {
        void* fn = nullptr;
        cudaDriverEntryPointQueryResult q;
        if (cudaGetDriverEntryPoint("cuTensorMapEncodeTiled", &fn, cudaEnableDefault, &q) != cudaSuccess || !fn) {
            zg_set_error("cuTensorMapEncodeTiled entry point not available");
            return false;
        }
        g_encode = (EncodeTiledFn)fn;
    }
    if (!g_attr_set) {
        cudaError_t e = cudaFuncSetAttribute(dense_gemm_kernel<false, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(dense_gemm_kernel<false, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
        if (e == cudaSuccess) e = cudaFuncSetAttribute(dense_gemm_kernel<true, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)kSmem);
        if (e != cudaSuccess) { zg_set_error("cudaFuncSetAttribute(dense_gemm) failed: %s", cudaGetErrorString(e)); return false; }
        g_attr_set = true;
    }
    return true;
}

}  // namespace

// The tensor path takes whole-tile-sized problems whose weight rows TMA can address (16-byte aligned base and pitch).
bool zg_dense_gemm_usable(const void* w_bf16, uint32_t M, uint32_t N, uint32_t K) {
    return M > 8 && N >= 8 && K >= 64 && K % 8 == 0 && (reinterpret_cast<uintptr_t>(w_bf16) & 15) == 0;
}
// bf16 copy of the activations: [round_up(M, 128)][round_up(K, 64)], counted in f32 slots
size_t zg_dense_gemm_scratch_elems(uint32_t M, uint32_t K) {
    return (size_t)((M + BM - 1) / BM * BM) * ((K + BK - 1) / BK * BK) / 2;
}
unsigned int zg_dense_gemm_timeouts() {
    unsigned int v = 0;
    cudaMemcpyFromSymbol(&v, g_timeouts, sizeof(v));
    return v;
}

bool zg_dense_gemm_launch(const void* w_bf16, const void* bias_bf16, const float* src, float* dst, uint32_t M, uint32_t N, uint32_t K,
                          uint32_t src_rs, uint32_t dst_rs, float* scratch, cudaStream_t st, uint32_t act, float act_p, const float* ctl, uint32_t slot_stride) {
    if (!prepare()) return false;
    const uint32_t Kp = (K + BK - 1) / BK * BK, Mp = (M + BM - 1) / BM * BM;
    uint32_t* xb = reinterpret_cast<uint32_t*>(scratch);
    k_to_bf16<<<dim3((Kp / 2 + 255) / 256, Mp), 256, 0, st>>>(src, src_rs, xb, Kp / 2, M, K, ctl, slot_stride);
    ZG_COUNT_LAUNCH();
    CUtensorMap map_a, map_b;
    const cuuint32_t estr[2] = {1, 1};
    {
        const cuuint64_t gdim[2] = {Kp, Mp};
        const cuuint64_t gstride[1] = {(cuuint64_t)Kp * 2};
        const cuuint32_t box[2] = {BK, BM};
        CUresult r = g_encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, xb, gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { zg_set_error("cuTensorMapEncodeTiled(activations) failed (%d)", (int)r); return false; }
    }
    {
        const cuuint64_t gdim[2] = {K, N};
        const cuuint64_t gstride[1] = {(cuuint64_t)K * 2};
        const cuuint32_t box[2] = {BK, BN};
        CUresult r = g_encode(&map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(w_bf16), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { zg_set_error("cuTensorMapEncodeTiled(weights) failed (%d)", (int)r); return false; }
    }
    GemmParams p;
    p.out = dst; p.bias = reinterpret_cast<const __nv_bfloat16*>(bias_bf16); p.M = M; p.N = N; p.K = K; p.out_rs = dst_rs; p.act = act; p.act_p = act_p;
    p.out_vec4 = ((reinterpret_cast<uintptr_t>(dst) & 15) == 0 && (dst_rs & 3) == 0) ? 1u : 0u;
    p.tile_group = nullptr;
    dim3 grid((N + BN - 1) / BN, (M + BM - 1) / BM);
    if (act) dense_gemm_kernel<false, true><<<grid, kThreads, kSmem, st>>>(map_a, map_b, p);
    else dense_gemm_kernel<false, false><<<grid, kThreads, kSmem, st>>>(map_a, map_b, p);
    ZG_COUNT_LAUNCH();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { zg_set_error("dense gemm launch failed: %s", cudaGetErrorString(e)); return false; }
    return true;
}

// Grouped form: xb = bf16 rows [rows][Kp] already sorted by group in whole 128-row tiles (rows % 128 == 0, Kp % 64 == 0, zero
// padding), W = [groups][N][K] bfloat16, dst[rows][N] f32.  d_tile_group[rows / 128] selects the matrix of every tile (< 0: skip).
bool zg_dense_gemm_grouped_launch(const void* w_bf16, uint32_t groups, const void* xb, uint32_t rows, uint32_t Kp, const int* d_tile_group, float* dst,
                                  uint32_t N, uint32_t K, uint32_t dst_rs, cudaStream_t st) {
    if (!prepare()) return false;
    CUtensorMap map_a, map_b;
    {
        const cuuint64_t gdim[2] = {Kp, rows};
        const cuuint64_t gstride[1] = {(cuuint64_t)Kp * 2};
        const cuuint32_t box[2] = {BK, BM}, estr[2] = {1, 1};
        CUresult r = g_encode(&map_a, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 2, const_cast<void*>(xb), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_128B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { zg_set_error("cuTensorMapEncodeTiled(grouped rows) failed (%d)", (int)r); return false; }
    }
    {
        const cuuint64_t gdim[3] = {K, N, groups};
        const cuuint64_t gstride[2] = {(cuuint64_t)K * 2, (cuuint64_t)N * K * 2};
        const cuuint32_t box[3] = {BK, BN, 1}, estr[3] = {1, 1, 1};
        CUresult r = g_encode(&map_b, CU_TENSOR_MAP_DATA_TYPE_BFLOAT16, 3, const_cast<void*>(w_bf16), gdim, gstride, box, estr, CU_TENSOR_MAP_INTERLEAVE_NONE,
                              CU_TENSOR_MAP_SWIZZLE_128B, CU_TENSOR_MAP_L2_PROMOTION_L2_256B, CU_TENSOR_MAP_FLOAT_OOB_FILL_NONE);
        if (r != CUDA_SUCCESS) { zg_set_error("cuTensorMapEncodeTiled(stacked weights) failed (%d)", (int)r); return false; }
    }
    GemmParams p;
    p.out = dst; p.bias = nullptr; p.M = rows; p.N = N; p.K = K; p.out_rs = dst_rs; p.act = 0; p.act_p = 0.0f;
    p.out_vec4 = ((reinterpret_cast<uintptr_t>(dst) & 15) == 0 && (dst_rs & 3) == 0) ? 1u : 0u;
    p.tile_group = d_tile_group;
    dim3 grid((N + BN - 1) / BN, rows / BM);
    dense_gemm_kernel<true, false><<<grid, kThreads, kSmem, st>>>(map_a, map_b, p);
    ZG_COUNT_LAUNCH();
    cudaError_t e = cudaGetLastError();
    if (e != cudaSuccess) { zg_set_error("grouped dense gemm launch failed: %s", cudaGetErrorString(e)); return false; }
    return true;
}
