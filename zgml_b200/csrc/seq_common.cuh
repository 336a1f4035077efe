// Helpers shared by the translation units of the sequence-model ops: weight loads of either format, warp and block
// reductions, programmatic dependent launch, the control words, and the launch-check macros of the dispatchers.
#pragma once
#include "zg_internal.cuh"

#include <cuda_bf16.h>

namespace {

typedef __nv_bfloat16 bf16;

template <typename WT> __device__ __forceinline__ float wld(const WT* w, size_t i);
template <> __device__ __forceinline__ float wld<float>(const float* w, size_t i) { return w[i]; }
template <> __device__ __forceinline__ float wld<bf16>(const bf16* w, size_t i) { return __bfloat162float(w[i]); }

__device__ __forceinline__ float warp_sum(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v += __shfl_xor_sync(0xffffffffu, v, o);
    return v;
}
__device__ __forceinline__ float warp_max(float v) {
#pragma unroll
    for (int o = 16; o > 0; o >>= 1) v = fmaxf(v, __shfl_xor_sync(0xffffffffu, v, o));
    return v;
}
// sum over the whole block, result in every thread; sh: 32 floats
__device__ float block_sum(float v, float* sh) {
    const int lane = threadIdx.x & 31, warp = threadIdx.x >> 5, nw = (blockDim.x + 31) >> 5;
    v = warp_sum(v);
    __syncthreads();
    if (lane == 0) sh[warp] = v;
    __syncthreads();
    float r = 0.0f;
    for (int i = 0; i < nw; i++) r += sh[i];
    return r;
}
// Programmatic dependent launch (as the framework's other program kernels do): let the next kernel of the stream become
// resident while this one runs, and hold this one until its predecessor has completed.  Nothing is read before the wait.
__device__ __forceinline__ void pdl_enter() {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    asm volatile("griddepcontrol.wait;" ::: "memory");
}
// `early` false: a plain launch, which starts when its predecessor has completed (for long kernels of few CTAs, whose placement
// should not be decided while the predecessor still fills the GPU)
template <typename... KArgs, typename... Args>
inline void launch_pdl_if(bool early, void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    cudaLaunchConfig_t cfg = {};
    cfg.gridDim = grid; cfg.blockDim = block; cfg.dynamicSmemBytes = smem; cfg.stream = st;
    cudaLaunchAttribute attr[1];
    attr[0].id = cudaLaunchAttributeProgrammaticStreamSerialization;
    attr[0].val.programmaticStreamSerializationAllowed = 1;
    cfg.attrs = attr;
    cfg.numAttrs = g_zg_pdl && early ? 1 : 0;
    cudaLaunchKernelEx(&cfg, kern, KArgs(args)...);
}
template <typename... KArgs, typename... Args>
inline void launch_pdl(void (*kern)(KArgs...), dim3 grid, dim3 block, size_t smem, cudaStream_t st, Args... args) {
    launch_pdl_if(true, kern, grid, block, smem, st, args...);
}
__device__ __forceinline__ float sigmoidf_(float z) { return 1.0f / (1.0f + expf(-z)); }
__device__ __forceinline__ float softplusf_(float z) { return z > 20.0f ? z : log1pf(expf(z)); }
__device__ __forceinline__ int ctl_word(const float* ctl, int i) { return reinterpret_cast<const int*>(ctl)[i]; }
// the activations of ACTIVATION and of LINEAR's epilogue: 0 relu(z)^2, 1 silu, 2 gelu (tanh form), 3 relu, 4 smooth cap
// p * tanh(z / p) (p: the op's activation parameter)
__device__ __forceinline__ float seq_activation(float z, uint32_t kind, float p = 0.0f) {
    switch (kind) {
        case 0: { const float r = fmaxf(z, 0.0f); return r * r; }
        case 1: return z * sigmoidf_(z);
        case 2: return 0.5f * z * (1.0f + tanhf(0.7978845608028654f * fmaf(0.044715f * z * z, z, z)));
        case 4: return p * tanhf(z / p);
        default: return fmaxf(z, 0.0f);
    }
}
// epilogue form: act = 0 none, kind + 1 otherwise
__device__ __forceinline__ float seq_epilogue(float z, uint32_t act, float p = 0.0f) { return act ? seq_activation(z, act - 1, p) : z; }

// 16-byte weight loads (8 bf16 / 4 f32 per lane and trip) when the row start and K allow it
template <typename WT> struct WVec;
template <> struct WVec<bf16> { static constexpr int n = 8; };
template <> struct WVec<float> { static constexpr int n = 4; };
template <typename WT>
__device__ __forceinline__ void wld_vec(const WT* p, float* out);
template <> __device__ __forceinline__ void wld_vec<bf16>(const bf16* p, float* out) {
    const uint4 v = *reinterpret_cast<const uint4*>(p);
    const uint32_t u[4] = {v.x, v.y, v.z, v.w};
#pragma unroll
    for (int i = 0; i < 4; i++) { out[2 * i] = __uint_as_float(u[i] << 16); out[2 * i + 1] = __uint_as_float(u[i] & 0xFFFF0000u); }
}
template <> __device__ __forceinline__ void wld_vec<float>(const float* p, float* out) {
    const float4 v = *reinterpret_cast<const float4*>(p);
    out[0] = v.x; out[1] = v.y; out[2] = v.z; out[3] = v.w;
}
template <typename WT> const WT* wptr(float* const* bufs, uint32_t b, uint32_t off) { return reinterpret_cast<const WT*>(bufs[b]) + off; }


}  // namespace

#define ZG_SEQ_CHECK()                                                                                          \
    do {                                                                                                        \
        cudaError_t _e = cudaGetLastError();                                                                    \
        if (_e != cudaSuccess) { zg_set_error("sequence op %u: launch failed: %s", op.tag, cudaGetErrorString(_e)); return false; } \
        ZG_COUNT_LAUNCH();                                                                                      \
    } while (0)
// run `call` with WT = the op's weight type
#define ZG_SEQ_WDT(wdt, ...)                                                          \
    do {                                                                              \
        if ((wdt) == ZG_W_BF16) { typedef bf16 WT; __VA_ARGS__; } else { typedef float WT; __VA_ARGS__; } \
    } while (0)

