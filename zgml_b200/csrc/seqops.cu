// Sequence-model DeviceOps (ZG_OP_EMBED .. ZG_OP_MOE_FFN, parameter packs documented in include/zgml_cuda.h): dense
// 16-bit / f32 weights against f32 activations, affine norms with a fused residual, windowed attention with a sink over a
// key ring, short causal convolutions with a carried tail, the gated delta-rule recurrence with per-channel decay, and a
// routed mixture of experts.  Everything is accumulated in f32; a bfloat16 weight is widened exactly on load, so the two
// weight formats differ only in bytes streamed.
//
// Per-sequence state lives in external program buffers indexed by the state slot of the control buffer; the position of
// the step's first token comes from the same place, so a captured graph replays unchanged from step to step.
#include "seq_common.cuh"

#include <stdlib.h>

namespace {

// ── EMBED ─────────────────────────────────────────────────────────────────────────────────────────────────────────
template <typename WT>
__global__ void k_embed(float* __restrict__ dst, const float* __restrict__ ctl, const WT* __restrict__ table, uint32_t D, float scale,
                        const WT* __restrict__ positions) {
    pdl_enter();
    const uint32_t t = blockIdx.x;
    const size_t row = (size_t)ctl_word(ctl, ZG_CTL_IDS + t) * D;
    if (positions) {       // a learned position row, not scaled
        const size_t prow = ((size_t)ctl_word(ctl, ZG_CTL_POS) + t) * D;
#pragma unroll 4
        for (uint32_t c = threadIdx.x; c < D; c += blockDim.x) dst[(size_t)t * D + c] = fmaf(wld(table, row + c), scale, wld(positions, prow + c));
        return;
    }
    for (uint32_t c = threadIdx.x; c < D; c += blockDim.x) dst[(size_t)t * D + c] = wld(table, row + c) * scale;
}

// ── LINEAR, few rows (decode): one warp per output feature, the weight row streamed once for all rows ─────────────────
constexpr int kGemvRows = 8;
template <typename WT>
__global__ void k_linear_rows(float* __restrict__ dst, const float* __restrict__ src, const WT* __restrict__ W, const WT* __restrict__ bias,
                              uint32_t M, uint32_t N, uint32_t K, uint32_t src_rs, uint32_t dst_rs, uint32_t act, float act_p, const float* __restrict__ ctl,
                              uint32_t slot_stride) {
    pdl_enter();
    if (ctl) src += (size_t)ctl_word(ctl, ZG_CTL_SLOT) * slot_stride;      // the rows of a per-sequence state buffer
    const uint32_t n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    const WT* w = W + (size_t)n * K;
    float acc[kGemvRows];
#pragma unroll
    for (int m = 0; m < kGemvRows; m++) acc[m] = 0.0f;
    for (uint32_t k = lane; k < K; k += 32) {
        const float wv = wld(w, k);
#pragma unroll
        for (int m = 0; m < kGemvRows; m++)
            if (m < (int)M) acc[m] = fmaf(src[(size_t)m * src_rs + k], wv, acc[m]);
    }
    const float b = bias ? wld(bias, n) : 0.0f;
#pragma unroll
    for (int m = 0; m < kGemvRows; m++) {
        if (m < (int)M) {
            const float s = warp_sum(acc[m]);
            if (lane == 0) dst[(size_t)m * dst_rs + n] = seq_epilogue(s + b, act, act_p);
        }
    }
}
// The activation rows are staged once per CTA in shared memory (float4 reads, no per-weight global loads); four weight
// vectors per lane are in flight per trip.
template <typename WT, int MR>
__global__ void k_linear_rows_vec(float* __restrict__ dst, const float* __restrict__ src, const WT* __restrict__ W, const WT* __restrict__ bias,
                                  uint32_t M, uint32_t N, uint32_t K, uint32_t src_rs, uint32_t dst_rs, uint32_t act, float act_p, const float* __restrict__ ctl,
                                  uint32_t slot_stride) {
    // Weights are constants of the model, so this warp's weight row is pulled toward L2 BEFORE the wait on the predecessor:
    // in a replayed graph the HBM stream of a matvec starts under the tail of the kernel that produces its input.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    {
        const uint32_t n0 = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5);
        if (n0 < N) {
            const char* wb = reinterpret_cast<const char*>(W + (size_t)n0 * K);
            for (size_t b = (size_t)(threadIdx.x & 31) * 128; b < (size_t)K * sizeof(WT); b += 32 * 128)
                asm volatile("prefetch.global.L2 [%0];" ::"l"(wb + b));
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    constexpr int V = WVec<WT>::n;
    extern __shared__ float xs[];                      // [M][K]
    if (ctl) src += (size_t)ctl_word(ctl, ZG_CTL_SLOT) * slot_stride;
    for (uint32_t e = threadIdx.x; e < M * K; e += blockDim.x) xs[e] = src[(size_t)(e / K) * src_rs + e % K];
    __syncthreads();
    const uint32_t n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (n >= N) return;
    const WT* w = W + (size_t)n * K;
    float acc[MR];
#pragma unroll
    for (int m = 0; m < MR; m++) acc[m] = 0.0f;
    auto fma_vec = [&](const float* wv, uint32_t k) {
#pragma unroll
        for (int m = 0; m < MR; m++) {
            if (m < (int)M) {
                const float4* x = reinterpret_cast<const float4*>(xs + (size_t)m * K + k);
#pragma unroll
                for (int i = 0; i < V / 4; i++) {
                    const float4 xv = x[i];
                    acc[m] = fmaf(xv.x, wv[4 * i], fmaf(xv.y, wv[4 * i + 1], fmaf(xv.z, wv[4 * i + 2], fmaf(xv.w, wv[4 * i + 3], acc[m]))));
                }
            }
        }
    };
    uint32_t k = lane * V;
    for (; k + 96 * V < K; k += 128 * V) {
        float w0[V], w1[V], w2[V], w3[V];
        wld_vec<WT>(w + k, w0);
        wld_vec<WT>(w + k + 32 * V, w1);
        wld_vec<WT>(w + k + 64 * V, w2);
        wld_vec<WT>(w + k + 96 * V, w3);
        fma_vec(w0, k);
        fma_vec(w1, k + 32 * V);
        fma_vec(w2, k + 64 * V);
        fma_vec(w3, k + 96 * V);
    }
    for (; k + 32 * V < K; k += 64 * V) {
        float w0[V], w1[V];
        wld_vec<WT>(w + k, w0);
        wld_vec<WT>(w + k + 32 * V, w1);
        fma_vec(w0, k);
        fma_vec(w1, k + 32 * V);
    }
    if (k < K) {
        float w0[V];
        wld_vec<WT>(w + k, w0);
        fma_vec(w0, k);
    }
    const float b = bias ? wld(bias, n) : 0.0f;
#pragma unroll
    for (int m = 0; m < MR; m++) {
        if (m < (int)M) {
            const float s = warp_sum(acc[m]);
            if (lane == 0) dst[(size_t)m * dst_rs + n] = seq_epilogue(s + b, act, act_p);
        }
    }
}

// ── LINEAR, many rows (prefill), exact f32: 64 x 64 tile, 16-deep k slices, 4 x 4 outputs per thread ──────────────────
constexpr int kTM = 64, kTN = 64, kTK = 16;
template <typename WT>
__global__ void __launch_bounds__(256) k_linear_tile(float* __restrict__ dst, const float* __restrict__ src, const WT* __restrict__ W,
                                                     const WT* __restrict__ bias, uint32_t M, uint32_t N, uint32_t K, uint32_t src_rs,
                                                     uint32_t dst_rs, uint32_t act, float act_p, const float* __restrict__ ctl, uint32_t slot_stride) {
    __shared__ float As[kTK][kTM + 4];
    __shared__ float Ws[kTK][kTN + 4];
    if (ctl) src += (size_t)ctl_word(ctl, ZG_CTL_SLOT) * slot_stride;
    const uint32_t m0 = blockIdx.y * kTM, n0 = blockIdx.x * kTN;
    const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;   // outputs: rows ty * 4 + i, columns tx * 4 + j
    float acc[4][4] = {};
    for (uint32_t k0 = 0; k0 < K; k0 += kTK) {
        for (uint32_t e = threadIdx.x; e < kTM * kTK; e += 256) {
            const uint32_t r = e / kTK, kk = e % kTK;
            const uint32_t m = m0 + r, k = k0 + kk;
            As[kk][r] = (m < M && k < K) ? src[(size_t)m * src_rs + k] : 0.0f;
            const uint32_t n = n0 + r;
            Ws[kk][r] = (n < N && k < K) ? wld(W, (size_t)n * K + k) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kTK; kk++) {
            float a[4], b[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { a[i] = As[kk][ty * 4 + i]; b[i] = Ws[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(a[i], b[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t m = m0 + ty * 4 + i;
        if (m >= M) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t n = n0 + tx * 4 + j;
            if (n < N) dst[(size_t)m * dst_rs + n] = seq_epilogue(acc[i][j] + (bias ? wld(bias, n) : 0.0f), act, act_p);
        }
    }
}

// ── NORM: one CTA per row ────────────────────────────────────────────────────────────────────────────────────────
// dst = (res +) norm(src; w) and, when a second destination is given, dst2 = norm(dst; w2) in the same launch: the norm
// that closes a sublayer (with the residual add) and the norm that opens the next one are one kernel.
constexpr int kNormCache = 16;   // values a thread keeps: rows up to 16 x blockDim are read from memory once
template <bool CACHED, typename WF>
__device__ __forceinline__ void norm_pass(float* __restrict__ out, const float* __restrict__ x, float (&v)[kNormCache], const float* __restrict__ res,
                                          const float (&rv)[kNormCache], uint32_t cols, uint32_t kind, float eps, float* sh, bool keep, WF wfn) {
    float s = 0.0f;
    if (CACHED) {
#pragma unroll
        for (int i = 0; i < kNormCache; i++) s += v[i];
    } else {
        for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) s += x[c];
    }
    const float mean = (kind & 1u) == 0 ? block_sum(s, sh) / (float)cols : 0.0f;
    float q = 0.0f;
    if (CACHED) {
#pragma unroll
        for (int i = 0; i < kNormCache; i++) {
            const uint32_t c = threadIdx.x + i * blockDim.x;
            const float d = c < cols ? v[i] - mean : 0.0f;
            q = fmaf(d, d, q);
        }
    } else {
        for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) { const float d = x[c] - mean; q = fmaf(d, d, q); }
    }
    const float inv = 1.0f / sqrtf(block_sum(q, sh) / (float)cols + eps);
    if (CACHED) {
#pragma unroll
        for (int i = 0; i < kNormCache; i++) {
            const uint32_t c = threadIdx.x + i * blockDim.x;
            if (c < cols) {
                const float y = (v[i] - mean) * inv * wfn(i, c);
                const float o = res ? rv[i] + y : y;
                out[c] = o;
                if (keep) v[i] = o;
            }
        }
    } else {
        for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
            const float y = (x[c] - mean) * inv * wfn(0, c);
            out[c] = res ? res[c] + y : y;
        }
    }
}
// weight as the norm applies it: stored around zero (kind bit 1) and / or carrying the gain of the product that follows (bit 2)
__device__ __forceinline__ float norm_weight(float w, uint32_t kind, float gain) {
    if (kind & 2u) w += 1.0f;
    return (kind & 4u) ? w * gain : w;
}
template <typename WT>
__global__ void k_norm(float* __restrict__ dst, const float* __restrict__ src, const WT* __restrict__ w, const float* __restrict__ res,
                       uint32_t cols, uint32_t kind, float eps, float* __restrict__ dst2, const WT* __restrict__ w2, uint32_t kind2, float gain,
                       const WT* __restrict__ shift_mix, float* __restrict__ shift_state, const float* __restrict__ ctl,
                       const WT* __restrict__ avg_coeff, uint32_t avg_terms, uint32_t avg_stride, float* __restrict__ avg_out) {
    // Rows that fit the registers: the norm weights are constants of the model and are read BEFORE the wait on the predecessor;
    // the row and the residual are read together right after it, so the kernel has one round of global loads, not three.
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float sh[32];
    const size_t row = (size_t)blockIdx.x * cols;
    const float* x = src + row;
    const bool cached = cols <= kNormCache * blockDim.x;
    float v[kNormCache], rv[kNormCache], wa[kNormCache], wb[kNormCache];
    if (cached) {
#pragma unroll
        for (int i = 0; i < kNormCache; i++) {
            const uint32_t c = threadIdx.x + i * blockDim.x;
            wa[i] = c < cols ? norm_weight(wld(w, c), kind, gain) : 0.0f;
            wb[i] = (dst2 && c < cols) ? norm_weight(wld(w2, c), kind2, gain) : 0.0f;
        }
    }
    asm volatile("griddepcontrol.wait;" ::: "memory");
    if (cached) {
        if (avg_terms) {   // the row to norm is a weighted sum of `avg_terms` streams (a depth average), kept in avg_out too
#pragma unroll
            for (int i = 0; i < kNormCache; i++) { v[i] = 0.0f; rv[i] = 0.0f; }
            for (uint32_t j = 0; j < avg_terms; j++) {     // one batch of independent loads per stream
                const float cj = wld(avg_coeff, j);
                const float* xj = x + (size_t)j * avg_stride;
#pragma unroll
                for (int i = 0; i < kNormCache; i++) {
                    const uint32_t c = threadIdx.x + i * blockDim.x;
                    if (c < cols) v[i] = fmaf(cj, xj[c], v[i]);
                }
            }
#pragma unroll
            for (int i = 0; i < kNormCache; i++) {
                const uint32_t c = threadIdx.x + i * blockDim.x;
                if (c < cols) avg_out[row + c] = v[i];
            }
        } else {
#pragma unroll
            for (int i = 0; i < kNormCache; i++) {
                const uint32_t c = threadIdx.x + i * blockDim.x;
                v[i] = c < cols ? x[c] : 0.0f;
                rv[i] = (res && c < cols) ? res[row + c] : 0.0f;
            }
        }
        norm_pass<true>(dst + row, x, v, res ? res + row : nullptr, rv, cols, kind, eps, sh, dst2 != nullptr, [&](int i, uint32_t) { return wa[i]; });
        if (dst2) norm_pass<true>(dst2 + row, dst + row, v, nullptr, rv, cols, kind2, eps, sh, false, [&](int i, uint32_t) { return wb[i]; });
    } else {
        if (avg_terms) {
            for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
                float acc = 0.0f;
                for (uint32_t j = 0; j < avg_terms; j++) acc = fmaf(wld(avg_coeff, j), x[(size_t)j * avg_stride + c], acc);
                avg_out[row + c] = acc;
            }
            __syncthreads();
            x = avg_out + row;
        }
        norm_pass<false>(dst + row, x, v, res ? res + row : nullptr, rv, cols, kind, eps, sh, false, [&](int, uint32_t c) { return norm_weight(wld(w, c), kind, gain); });
        if (dst2) {
            __syncthreads();                           // the row just written is read back by other threads
            norm_pass<false>(dst2 + row, dst + row, v, nullptr, rv, cols, kind2, eps, sh, false, [&](int, uint32_t c) { return norm_weight(wld(w2, c), kind2, gain); });
        }
    }
    // Single-row steps: the token shift of the launch's last output happens here too.  Every thread revisits the columns it
    // wrote itself, so no barrier is needed; the state keeps the row as it was before the shift.
    if (shift_state) {
        float* st = shift_state + (size_t)ctl_word(ctl, ZG_CTL_SLOT) * cols;
        float* last = dst2 ? dst2 : dst;
        for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
            const float h = last[row + c], prev = st[c];
            st[c] = h;
            last[row + c] = fmaf(prev - h, wld(shift_mix, c), h);
        }
    }
}

// Kinds without row statistics (Dynamic Tanh; the plain residual step), their combinations with the others, and the sum of TWO
// normed sources: one CTA per row.  dst = (res +) f(src) (+ f_b(src_b)) and, with dst2, dst2 = f2(dst): the residual step that
// closes a sublayer and the Dynamic Tanh that opens the next are one launch.  Rows of up to kNormCache x blockDim values live in
// registers: weights and biases are constants of the model and are read BEFORE the wait on the predecessor, the row, its
// residual and the second source together right after it.  Wider rows are walked from memory.
template <typename WT>
__device__ __forceinline__ float norm_any_value(float x, float mean, float inv, float w, float aux, uint32_t kind, float gain, float alpha) {
    const float g = (kind & 4u) ? gain : 1.0f;
    if (kind & 16u) return x * g;
    if (kind & 8u) return fmaf(tanhf(alpha * x), w, aux) * g;
    return (x - mean) * inv * ((kind & 2u) ? w + 1.0f : w) * g;
}
template <typename WT>
__device__ void norm_any_pass(float* out, const float* x, const float* res, const WT* __restrict__ w, uint32_t cols, uint32_t kind, float eps, float gain,
                              float* sh, const float* xb, const WT* __restrict__ wb) {
    float mean = 0.0f, inv = 1.0f, mean_b = 0.0f, inv_b = 1.0f;
    if (!(kind & 24u)) {
        if (!(kind & 1u)) {
            float sum = 0.0f, sum_b = 0.0f;
            for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) { sum += x[c]; if (xb) sum_b += xb[c]; }
            mean = block_sum(sum, sh) / (float)cols;
            if (xb) mean_b = block_sum(sum_b, sh) / (float)cols;
        }
        float q = 0.0f, qb = 0.0f;
        for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
            const float d = x[c] - mean; q = fmaf(d, d, q);
            if (xb) { const float e = xb[c] - mean_b; qb = fmaf(e, e, qb); }
        }
        inv = 1.0f / sqrtf(block_sum(q, sh) / (float)cols + eps);
        if (xb) inv_b = 1.0f / sqrtf(block_sum(qb, sh) / (float)cols + eps);
    }
    const float alpha = (kind & 8u) ? wld(w, (size_t)2 * cols) : 0.0f;
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
        float y = norm_any_value<WT>(x[c], mean, inv, (kind & 16u) ? 0.0f : wld(w, c), (kind & 8u) ? wld(w, (size_t)cols + c) : 0.0f, kind, gain, alpha);
        if (xb) y += norm_any_value<WT>(xb[c], mean_b, inv_b, wld(wb, c), 0.0f, kind, gain, 0.0f);
        out[c] = res ? res[c] + y : y;
    }
}
// many rows (prompts): what counts is how many rows are resident per SM, so nothing is kept in registers
template <typename WT>
__global__ void __launch_bounds__(256) k_norm_any_rows(float* dst, const float* src, const WT* __restrict__ w, const float* res, uint32_t cols, uint32_t kind, float eps,
                                                       float* dst2, const WT* __restrict__ w2, uint32_t kind2, float gain, const float* src_b, const WT* __restrict__ w_b) {
    pdl_enter();
    __shared__ float sh[32];
    const size_t row = (size_t)blockIdx.x * cols;
    norm_any_pass(dst + row, src + row, res ? res + row : nullptr, w, cols, kind, eps, gain, sh, src_b ? src_b + row : nullptr, w_b);
    if (dst2) {
        __syncthreads();                                   // the row just written is read back by other threads
        norm_any_pass(dst2 + row, dst + row, (const float*)nullptr, w2, cols, kind2, eps, gain, sh, (const float*)nullptr, (const WT*)nullptr);
    }
}
template <typename WT, int kKeep, int kThreads>          // a row of up to kKeep x kThreads values lives in registers (fewer kept values, more CTAs per SM)
__global__ void __launch_bounds__(kThreads) k_norm_any(float* dst, const float* src, const WT* __restrict__ w, const float* res, uint32_t cols, uint32_t kind, float eps,
                                                  float* dst2, const WT* __restrict__ w2, uint32_t kind2, float gain, const float* src_b, const WT* __restrict__ w_b) {
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    __shared__ float sh[32];
    const size_t row = (size_t)blockIdx.x * cols;
    if (cols > kKeep * kThreads) {                  // rows too wide for the registers
        asm volatile("griddepcontrol.wait;" ::: "memory");
        norm_any_pass(dst + row, src + row, res ? res + row : nullptr, w, cols, kind, eps, gain, sh, src_b ? src_b + row : nullptr, w_b);
        if (dst2) {
            __syncthreads();                               // the row just written is read back by other threads
            norm_any_pass(dst2 + row, dst + row, (const float*)nullptr, w2, cols, kind2, eps, gain, sh, (const float*)nullptr, (const WT*)nullptr);
        }
        return;
    }
    float v[kKeep], wa[kKeep], aux[kKeep], wc[kKeep], bc[kKeep];   // aux: the bias of a Dynamic Tanh, or the second source's weight
#pragma unroll
    for (int i = 0; i < kKeep; i++) {
        const uint32_t c = threadIdx.x + i * blockDim.x;
        const bool in = c < cols;
        wa[i] = (in && !(kind & 16u)) ? wld(w, c) : 0.0f;
        aux[i] = in ? ((kind & 8u) ? wld(w, (size_t)cols + c) : (src_b ? wld(w_b, c) : 0.0f)) : 0.0f;
        wc[i] = (in && dst2 && !(kind2 & 16u)) ? wld(w2, c) : 0.0f;
        bc[i] = (in && dst2 && (kind2 & 8u)) ? wld(w2, (size_t)cols + c) : 0.0f;
    }
    const float alpha = (kind & 8u) ? wld(w, (size_t)2 * cols) : 0.0f, alpha2 = (dst2 && (kind2 & 8u)) ? wld(w2, (size_t)2 * cols) : 0.0f;
    asm volatile("griddepcontrol.wait;" ::: "memory");
    float rv[kKeep], vb[kKeep];
#pragma unroll
    for (int i = 0; i < kKeep; i++) {
        const uint32_t c = threadIdx.x + i * blockDim.x;
        v[i] = c < cols ? src[row + c] : 0.0f;
        rv[i] = (res && c < cols) ? res[row + c] : 0.0f;
        vb[i] = (src_b && c < cols) ? src_b[row + c] : 0.0f;
    }
    auto stats = [&](const float (&val)[kKeep], uint32_t k, float& mean, float& inv) {
        mean = 0.0f; inv = 1.0f;
        if (k & 24u) return;
        if (!(k & 1u)) {
            float sum = 0.0f;
#pragma unroll
            for (int i = 0; i < kKeep; i++) sum += val[i];
            mean = block_sum(sum, sh) / (float)cols;
        }
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < kKeep; i++) {
            const float d = threadIdx.x + i * blockDim.x < cols ? val[i] - mean : 0.0f;
            q = fmaf(d, d, q);
        }
        inv = 1.0f / sqrtf(block_sum(q, sh) / (float)cols + eps);
    };
    float mean, inv, mean_b = 0.0f, inv_b = 1.0f;
    stats(v, kind, mean, inv);
    if (src_b) stats(vb, kind, mean_b, inv_b);
#pragma unroll
    for (int i = 0; i < kKeep; i++) {
        const uint32_t c = threadIdx.x + i * blockDim.x;
        float y = norm_any_value<WT>(v[i], mean, inv, wa[i], aux[i], kind, gain, alpha);
        if (src_b) y += norm_any_value<WT>(vb[i], mean_b, inv_b, aux[i], 0.0f, kind, gain, 0.0f);
        v[i] = res ? rv[i] + y : y;
        if (c < cols) dst[row + c] = v[i];
    }
    if (!dst2) return;
    stats(v, kind2, mean, inv);
#pragma unroll
    for (int i = 0; i < kKeep; i++) {
        const uint32_t c = threadIdx.x + i * blockDim.x;
        if (c < cols) dst2[row + c] = norm_any_value<WT>(v[i], mean, inv, wc[i], bc[i], kind2, gain, alpha2);
    }
}

// ── WINDOW_ATTENTION ─────────────────────────────────────────────────────────────────────────────────────────────
__global__ void k_ring_append(float* __restrict__ ring, const float* __restrict__ proj, const float* __restrict__ ctl, uint32_t k_off,
                              uint32_t proj_rs, uint32_t width, uint32_t R) {
    pdl_enter();
    const uint32_t t = blockIdx.x;
    const uint32_t pos = (uint32_t)ctl_word(ctl, ZG_CTL_POS) + t, slot = (uint32_t)ctl_word(ctl, ZG_CTL_SLOT);
    float* row = ring + ((size_t)slot * R + pos % R) * width;
    const float* k = proj + (size_t)t * proj_rs + k_off;
    for (uint32_t c = threadIdx.x; c < width; c += blockDim.x) row[c] = k[c];
}
constexpr int kAttnMaxDim = 256;   // 8 channels per lane
// one warp per (token, head): 32 keys at a time, lane = key for the scores, lane = channel for the weighted sum
__global__ void k_window_attention(float* __restrict__ dst, const float* __restrict__ proj, const float* __restrict__ ring,
                                   const float* __restrict__ bias, const float* __restrict__ ctl, uint32_t T, uint32_t H, uint32_t G,
                                   uint32_t dim, uint32_t proj_rs, uint32_t q_off, uint32_t g_off, uint32_t window, uint32_t R,
                                   float scale, float cap) {
    pdl_enter();
    extern __shared__ float sq[];                      // [warps][dim]
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const uint32_t item = blockIdx.x * nw + warp;
    if (item >= T * H) return;
    const uint32_t t = item / H, h = item % H, kv = h / (H / G);
    const uint32_t pos0 = (uint32_t)ctl_word(ctl, ZG_CTL_POS), slot = (uint32_t)ctl_word(ctl, ZG_CTL_SLOT);
    const uint32_t p = pos0 + t;
    const uint32_t lo = p + 1 >= window ? p + 1 - window : 0;
    float* q = sq + warp * dim;
    const float* qrow = proj + (size_t)t * proj_rs + q_off + (size_t)h * dim;
    for (uint32_t c = lane; c < dim; c += 32) q[c] = qrow[c];
    __syncwarp();
    const size_t width = (size_t)G * dim;
    const float* base = ring + (size_t)slot * R * width + (size_t)kv * dim;
    float m = 0.0f, l = 1.0f;                          // the sink: score 0, weight exp(0 - m), no value
    float acc[kAttnMaxDim / 32];
#pragma unroll
    for (int i = 0; i < kAttnMaxDim / 32; i++) acc[i] = 0.0f;
    for (uint32_t j0 = lo; j0 <= p; j0 += 32) {
        const uint32_t j = j0 + lane;
        float s = -INFINITY;
        if (j <= p) {
            const float* k = base + (size_t)(j % R) * width;
            float d = 0.0f;
            for (uint32_t c = 0; c < dim; c++) d = fmaf(q[c], k[c], d);
            s = d * scale;
            if (cap > 0.0f) s = cap * tanhf(s / cap);
            s += bias[(size_t)(p - j) * H + h];
        }
        const float m_new = fmaxf(m, warp_max(s));
        const float corr = expf(m - m_new);
        const float e = j <= p ? expf(s - m_new) : 0.0f;
        l = l * corr + warp_sum(e);
        m = m_new;
        const uint32_t cnt = min(32u, p - j0 + 1);
#pragma unroll
        for (int i = 0; i < kAttnMaxDim / 32; i++) acc[i] *= corr;
        for (uint32_t jj = 0; jj < cnt; jj++) {
            const float pj = __shfl_sync(0xffffffffu, e, jj);
            const float* k = base + (size_t)((j0 + jj) % R) * width;
#pragma unroll
            for (int i = 0; i < kAttnMaxDim / 32; i++) {
                const uint32_t c = lane + 32 * i;
                if (c < dim) acc[i] = fmaf(pj, k[c], acc[i]);
            }
        }
    }
    const float inv = 1.0f / l;
    const float* grow = proj + (size_t)t * proj_rs + g_off + (size_t)h * dim;
    float* out = dst + ((size_t)t * H + h) * dim;
#pragma unroll
    for (int i = 0; i < kAttnMaxDim / 32; i++) {
        const uint32_t c = lane + 32 * i;
        if (c < dim) out[c] = acc[i] * inv * sigmoidf_(grow[c]);
    }
}

// The kernel above is the fallback for head sizes that are not a multiple of 4.  This one: one CTA per (token, head), its
// warps split the window; inside a warp LK lanes share a key (each holds 4 * CH channels of it as float4s, so a key row is
// one coalesced read that serves the score AND — keys being the values — the weighted sum), 32 / LK keys per trip.  Every
// lane group keeps its own running (max, sum, accumulator); groups and warps are merged at the end, where the sink joins.
template <int CH>
__global__ void k_window_attention_v(float* __restrict__ dst, const float* __restrict__ proj, const float* __restrict__ ring,
                                     const float* __restrict__ bias, const float* __restrict__ ctl, uint32_t H, uint32_t G, uint32_t dim,
                                     uint32_t LK, uint32_t proj_rs, uint32_t q_off, uint32_t g_off, uint32_t window, uint32_t R, float scale,
                                     float cap, float* __restrict__ part) {
    pdl_enter();
    extern __shared__ float sm[];                      // [warps][4 + dim]: max, sum, two pad words (float4 alignment), accumulator
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const uint32_t t = blockIdx.x / H, h = blockIdx.x % H, kv = h / (H / G);
    const uint32_t pos0 = (uint32_t)ctl_word(ctl, ZG_CTL_POS), slot = (uint32_t)ctl_word(ctl, ZG_CTL_SLOT);
    const uint32_t p = pos0 + t;
    const uint32_t lo = p + 1 >= window ? p + 1 - window : 0;
    const uint32_t KP = 32 / LK, sub = lane % LK, ks = lane / LK;
    const float* qrow = proj + (size_t)t * proj_rs + q_off + (size_t)h * dim;
    float4 q[CH], acc[CH];
    bool valid[CH];
#pragma unroll
    for (int c = 0; c < CH; c++) {
        const uint32_t ch = (c * LK + sub) * 4;
        valid[c] = ch < dim;
        q[c] = valid[c] ? *reinterpret_cast<const float4*>(qrow + ch) : make_float4(0, 0, 0, 0);
        acc[c] = make_float4(0, 0, 0, 0);
    }
    const size_t width = (size_t)G * dim;
    const float* base = ring + (size_t)slot * R * width + (size_t)kv * dim;
    // gridDim.y CTAs split the window (decode: few (token, head) pairs, long windows), the warps of a CTA split its share
    const uint32_t n_keys = p - lo + 1;
    const uint32_t per_cta = (n_keys + gridDim.y - 1) / gridDim.y;
    const uint32_t c_begin = lo + blockIdx.y * per_cta, c_end = min(p + 1, c_begin + per_cta);
    const uint32_t per = ((c_end > c_begin ? c_end - c_begin : 0) + nw - 1) / nw;
    const uint32_t j_begin = c_begin + warp * per, j_end = min(c_end, j_begin + per);   // this warp's keys [j_begin, j_end)
    float m = -INFINITY, l = 0.0f;
    constexpr int U = 4;                               // keys in flight per lane group: their loads are issued together
    for (uint32_t j0 = j_begin; j0 < j_end; j0 += KP * U) {
        float4 kvv[U][CH];
        float d[U], bj[U];                             // the distance biases travel with the keys: no load inside the serial softmax update
        bool on[U];
#pragma unroll
        for (int u = 0; u < U; u++) {
            const uint32_t j = j0 + u * KP + ks;
            on[u] = j < j_end;
            bj[u] = on[u] ? bias[(size_t)(p - j) * H + h] : 0.0f;
            const float* k = base + (size_t)(j % R) * width;
#pragma unroll
            for (int c = 0; c < CH; c++)
                kvv[u][c] = (on[u] && valid[c]) ? *reinterpret_cast<const float4*>(k + (c * LK + sub) * 4) : make_float4(0, 0, 0, 0);
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            d[u] = 0.0f;
#pragma unroll
            for (int c = 0; c < CH; c++)
                d[u] = fmaf(q[c].x, kvv[u][c].x, fmaf(q[c].y, kvv[u][c].y, fmaf(q[c].z, kvv[u][c].z, fmaf(q[c].w, kvv[u][c].w, d[u]))));
        }
        for (uint32_t o = LK >> 1; o > 0; o >>= 1) {
#pragma unroll
            for (int u = 0; u < U; u++) d[u] += __shfl_xor_sync(0xffffffffu, d[u], o);
        }
#pragma unroll
        for (int u = 0; u < U; u++) {
            if (!on[u]) continue;
            float sc = d[u] * scale;
            if (cap > 0.0f) sc = cap * tanhf(sc / cap);
            sc += bj[u];
            if (sc > m) {
                const float corr = expf(m - sc);        // exp(-inf) = 0 on the first key
                l *= corr;
#pragma unroll
                for (int c = 0; c < CH; c++) { acc[c].x *= corr; acc[c].y *= corr; acc[c].z *= corr; acc[c].w *= corr; }
                m = sc;
            }
            const float pj = expf(sc - m);
            l += pj;
#pragma unroll
            for (int c = 0; c < CH; c++) {
                acc[c].x = fmaf(pj, kvv[u][c].x, acc[c].x); acc[c].y = fmaf(pj, kvv[u][c].y, acc[c].y);
                acc[c].z = fmaf(pj, kvv[u][c].z, acc[c].z); acc[c].w = fmaf(pj, kvv[u][c].w, acc[c].w);
            }
        }
    }
    // merge the key slots of the warp (lanes that differ in lane / LK)
    for (uint32_t o = LK; o < 32; o <<= 1) {
        const float m2 = __shfl_xor_sync(0xffffffffu, m, o), l2 = __shfl_xor_sync(0xffffffffu, l, o);
        const float M = fmaxf(m, m2);
        const float w1 = m == -INFINITY ? 0.0f : expf(m - M), w2 = m2 == -INFINITY ? 0.0f : expf(m2 - M);
        l = l * w1 + l2 * w2;
#pragma unroll
        for (int c = 0; c < CH; c++) {
            acc[c].x = acc[c].x * w1 + __shfl_xor_sync(0xffffffffu, acc[c].x, o) * w2;
            acc[c].y = acc[c].y * w1 + __shfl_xor_sync(0xffffffffu, acc[c].y, o) * w2;
            acc[c].z = acc[c].z * w1 + __shfl_xor_sync(0xffffffffu, acc[c].z, o) * w2;
            acc[c].w = acc[c].w * w1 + __shfl_xor_sync(0xffffffffu, acc[c].w, o) * w2;
        }
        m = M;
    }
    float* mine = sm + warp * (4 + dim);
    if (lane < LK) {
        if (sub == 0) { mine[0] = m; mine[1] = l; }
#pragma unroll
        for (int c = 0; c < CH; c++)
            if (valid[c]) *reinterpret_cast<float4*>(mine + 4 + (c * LK + sub) * 4) = acc[c];
    }
    __syncthreads();
    // merge the warps
    float M = -INFINITY;
    for (uint32_t w = 0; w < nw; w++) M = fmaxf(M, sm[w * (4 + dim)]);
    float L = 0.0f;
    for (uint32_t w = 0; w < nw; w++) { const float mw = sm[w * (4 + dim)]; if (mw != -INFINITY) L += sm[w * (4 + dim) + 1] * expf(mw - M); }
    const float* grow = proj + (size_t)t * proj_rs + g_off + (size_t)h * dim;
    float* out = dst + ((size_t)t * H + h) * dim;
    float* mine_part = part ? part + ((size_t)blockIdx.x * gridDim.y + blockIdx.y) * (4 + dim) : nullptr;
    // the sink (score 0, no value) joins the denominator where the last merge happens
    const float Ms = fmaxf(M, 0.0f);
    const float wk = M == -INFINITY ? 0.0f : expf(M - Ms);
    const float inv = 1.0f / (expf(-Ms) + L * wk);
    if (mine_part && threadIdx.x == 0) { mine_part[0] = M; mine_part[1] = L; }
    for (uint32_t c = threadIdx.x; c < dim; c += blockDim.x) {
        float a = 0.0f;
        for (uint32_t w = 0; w < nw; w++) { const float mw = sm[w * (4 + dim)]; if (mw != -INFINITY) a = fmaf(sm[w * (4 + dim) + 4 + c], expf(mw - M), a); }
        if (mine_part) mine_part[4 + c] = a;
        else out[c] = a * wk * inv * sigmoidf_(grow[c]);
    }
}
// merge of the window shares of k_window_attention_v: one CTA per (token, head)
__global__ void k_window_attention_merge(float* __restrict__ dst, const float* __restrict__ proj, const float* __restrict__ part, uint32_t H, uint32_t dim,
                                         uint32_t S, uint32_t proj_rs, uint32_t g_off) {
    pdl_enter();
    const uint32_t t = blockIdx.x / H, h = blockIdx.x % H;
    const float* P = part + (size_t)blockIdx.x * S * (4 + dim);
    float M = 0.0f;                                    // the sink's score
    for (uint32_t i = 0; i < S; i++) M = fmaxf(M, P[i * (4 + dim)]);
    float L = expf(-M);
    for (uint32_t i = 0; i < S; i++) { const float mi = P[i * (4 + dim)]; if (mi != -INFINITY) L += P[i * (4 + dim) + 1] * expf(mi - M); }
    const float inv = 1.0f / L;
    const float* grow = proj + (size_t)t * proj_rs + g_off + (size_t)h * dim;
    for (uint32_t c = threadIdx.x; c < dim; c += blockDim.x) {
        float a = 0.0f;
        for (uint32_t i = 0; i < S; i++) { const float mi = P[i * (4 + dim)]; if (mi != -INFINITY) a = fmaf(P[i * (4 + dim) + 4 + c], expf(mi - M), a); }
        dst[((size_t)t * H + h) * dim + c] = a * inv * sigmoidf_(grow[c]);
    }
}

// Prefill form of WINDOW_ATTENTION (16 or more tokens, head size up to 128): flash tiling in f32, as the framework's causal
// prefill attention does.  One CTA owns 64 consecutive queries of one head and walks the keys its window reaches in tiles
// of 64 ring rows.  The key tile in shared memory serves the scores AND, keys being the values, the weighted sum.  Thread
// (ty, tx) of 16 x 16 holds queries 4 ty .. 4 ty + 3 against keys tx + 16 c (conflict-free float4 reads of padded key rows);
// the row statistics of the running softmax are shared by the 16 threads of a row through half-warp shuffles; the
// probabilities pass through shared memory; outputs tx + 16 c of the four rows accumulate in registers.  The distance
// biases a tile can meet (127 distances) are staged once per tile, -inf standing for "outside the window or the future".
// The sink joins the denominator at the end, then the output gate.  DH = 16 OC covers the head; channels past dim are zero.
constexpr int kWaBQ = 64, kWaBK = 64, kWaThreads = 256, kWaTiledMinTokens = 16;
template <int OC>
__global__ void __launch_bounds__(kWaThreads, 2)
k_window_attention_tiled(float* __restrict__ dst, const float* __restrict__ proj, const float* __restrict__ ring, const float* __restrict__ bias,
                         const float* __restrict__ ctl, uint32_t T, uint32_t H, uint32_t G, uint32_t dim, uint32_t proj_rs, uint32_t q_off,
                         uint32_t g_off, uint32_t window, uint32_t R, float scale, float cap, uint32_t n_sm) {
    pdl_enter();
    constexpr int DH = 16 * OC, KP = DH + 4, PP = kWaBK + 4;
    extern __shared__ __align__(16) float sm[];
    float* Qs = sm;                                    // [64][DH]
    float* Ks = Qs + kWaBQ * DH;                       // [64][DH + 4]
    float* Ps = Ks + kWaBK * KP;                       // [64][64 + 4]
    float* Bs = Ps + kWaBQ * PP;                       // [128]
    // A later query tile walks more key tiles.  Blocks are ranked heaviest first (the block scheduler hands them out in index
    // order); when the whole grid is resident at once, two CTAs per SM, the second CTA of every SM is taken from the light
    // end instead, so that each SM's pair carries about the same number of key tiles.
    uint32_t rank = blockIdx.x;
    if (gridDim.x <= 2 * n_sm && rank >= n_sm) rank = gridDim.x - 1 - (rank - n_sm);
    const uint32_t n_tiles = (T + kWaBQ - 1) / kWaBQ;
    const uint32_t h = rank % H, kv = h / (H / G), t0 = (n_tiles - 1 - rank / H) * kWaBQ;
    const uint32_t tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const uint32_t pos0 = (uint32_t)ctl_word(ctl, ZG_CTL_POS), slot = (uint32_t)ctl_word(ctl, ZG_CTL_SLOT);
    const uint32_t nq = min((uint32_t)kWaBQ, T - t0);
    const uint32_t p_first = pos0 + t0, p_last = p_first + nq - 1;
    const uint32_t lo = p_first + 1 >= window ? p_first + 1 - window : 0;
    const size_t width = (size_t)G * dim;
    const float* base = ring + (size_t)slot * R * width + (size_t)kv * dim;
    for (uint32_t i = tid; i < kWaBQ * (DH / 4); i += kWaThreads) {
        const uint32_t r = i / (DH / 4), c4 = i % (DH / 4);
        float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
        if (r < nq && 4 * c4 < dim) val = *reinterpret_cast<const float4*>(proj + (size_t)(t0 + r) * proj_rs + q_off + (size_t)h * dim + 4 * c4);
        *reinterpret_cast<float4*>(Qs + r * DH + 4 * c4) = val;
    }
    float o[4][OC], m_run[4], l_run[4];
#pragma unroll
    for (int r = 0; r < 4; r++) {
        m_run[r] = -INFINITY; l_run[r] = 0.0f;
#pragma unroll
        for (int c = 0; c < OC; c++) o[r][c] = 0.0f;
    }
    for (uint32_t s0 = lo; s0 <= p_last; s0 += kWaBK) {
        __syncthreads();                               // the previous tile's readers of Ks / Ps / Bs are done
        for (uint32_t i = tid; i < kWaBK * (DH / 4); i += kWaThreads) {
            const uint32_t r = i / (DH / 4), c4 = i % (DH / 4);
            float4 val = make_float4(0.f, 0.f, 0.f, 0.f);
            if (s0 + r <= p_last && 4 * c4 < dim) val = *reinterpret_cast<const float4*>(base + (size_t)((s0 + r) % R) * width + 4 * c4);
            *reinterpret_cast<float4*>(Ks + r * KP + 4 * c4) = val;
        }
        if (tid < 2 * kWaBK - 1) {                     // distance of (query row a, key column b) = p_first - s0 + a - b
            const int d = (int)p_first - (int)s0 - (kWaBK - 1) + (int)tid;
            Bs[tid] = (d >= 0 && d < (int)window) ? bias[(size_t)d * H + h] : -INFINITY;
        }
        __syncthreads();
        float sc[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int c = 0; c < 4; c++) sc[r][c] = 0.0f;
#pragma unroll 2
        for (int d = 0; d < DH; d += 4) {
            float4 qa[4], ka[4];
#pragma unroll
            for (int r = 0; r < 4; r++) qa[r] = *reinterpret_cast<const float4*>(Qs + (4 * ty + r) * DH + d);
#pragma unroll
            for (int c = 0; c < 4; c++) ka[c] = *reinterpret_cast<const float4*>(Ks + (tx + 16 * c) * KP + d);
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) {
                    sc[r][c] = fmaf(qa[r].x, ka[c].x, sc[r][c]); sc[r][c] = fmaf(qa[r].y, ka[c].y, sc[r][c]);
                    sc[r][c] = fmaf(qa[r].z, ka[c].z, sc[r][c]); sc[r][c] = fmaf(qa[r].w, ka[c].w, sc[r][c]);
                }
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const uint32_t a = 4 * ty + r;
            float rmax = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float b = Bs[a + (kWaBK - 1) - (tx + 16 * c)];
                float sv = -INFINITY;
                if (a < nq && b != -INFINITY) {
                    sv = sc[r][c] * scale;
                    if (cap > 0.0f) sv = cap * tanhf(sv / cap);
                    sv += b;
                }
                sc[r][c] = sv;
                rmax = fmaxf(rmax, sv);
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, off));
            const float new_m = fmaxf(m_run[r], rmax);
            const float alpha = m_run[r] == -INFINITY ? (new_m == -INFINITY ? 1.0f : 0.0f) : expf(m_run[r] - new_m);
            float rsum = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float pv = sc[r][c] == -INFINITY ? 0.0f : expf(sc[r][c] - new_m);
                Ps[a * PP + tx + 16 * c] = pv;
                rsum += pv;
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) rsum += __shfl_xor_sync(0xffffffffu, rsum, off);
            l_run[r] = l_run[r] * alpha + rsum;
            m_run[r] = new_m;
#pragma unroll
            for (int c = 0; c < OC; c++) o[r][c] *= alpha;
        }
        __syncthreads();
#pragma unroll 4
        for (int j = 0; j < kWaBK; j++) {
            float pj[4], vj[OC];
#pragma unroll
            for (int r = 0; r < 4; r++) pj[r] = Ps[(4 * ty + r) * PP + j];
#pragma unroll
            for (int c = 0; c < OC; c++) vj[c] = Ks[j * KP + tx + 16 * c];
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < OC; c++) o[r][c] = fmaf(pj[r], vj[c], o[r][c]);
        }
    }
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const uint32_t a = 4 * ty + r;
        if (a >= nq) continue;
        // every query sees itself, so m_run is finite; the sink (score 0, no value) joins the denominator here
        const float Ms = fmaxf(m_run[r], 0.0f);
        const float wk = expf(m_run[r] - Ms);
        const float inv = wk / (expf(-Ms) + l_run[r] * wk);
        const float* grow = proj + (size_t)(t0 + a) * proj_rs + g_off + (size_t)h * dim;
        float* out = dst + ((size_t)(t0 + a) * H + h) * dim;
#pragma unroll
        for (int c = 0; c < OC; c++) {
            const uint32_t col = tx + 16 * c;
            if (col < dim) out[col] = o[r][c] * inv * sigmoidf_(grow[col]);
        }
    }
}
template <int OC>
static void launch_window_attention_tiled(const ZgSeqOp& s, float* const* bufs, cudaStream_t st) {
    constexpr int DH = 16 * OC;
    const size_t smem = ((size_t)kWaBQ * DH + (size_t)kWaBK * (DH + 4) + (size_t)kWaBQ * (kWaBK + 4) + 2 * kWaBK) * sizeof(float);
    static bool once = false;
    if (!once) { cudaFuncSetAttribute(k_window_attention_tiled<OC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); once = true; }
    static int n_sm = 0;
    if (!n_sm) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev); if (n_sm <= 0) n_sm = 1; }
    launch_pdl(k_window_attention_tiled<OC>, dim3(((s.n[0] + kWaBQ - 1) / kWaBQ) * s.n[1]), dim3(kWaThreads), smem, st, bufs[s.buf[0]], bufs[s.buf[1]], bufs[s.buf[2]],
               bufs[s.buf[3]], bufs[s.buf[4]], s.n[0], s.n[1], s.n[2], s.n[3], s.n[4], s.off[0], s.off[2], s.n[5], s.n[6], s.f[0], s.f[1], (uint32_t)n_sm);
}

// ── CAUSAL_CONV ──────────────────────────────────────────────────────────────────────────────────────────────────
template <typename WT>
__global__ void k_causal_conv(float* __restrict__ dst, const float* __restrict__ src, const WT* __restrict__ w, float* state,
                              const float* __restrict__ ctl, uint32_t T, uint32_t C, uint32_t taps, uint32_t src_rs, uint32_t dst_rs, uint32_t act,
                              uint32_t advance, const WT* __restrict__ bias) {
    pdl_enter();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (size_t)T * C) return;
    const uint32_t t = (uint32_t)(e / C), c = (uint32_t)(e % C);
    float* st = state + (size_t)ctl_word(ctl, ZG_CTL_SLOT) * (taps - 1) * C;
    float y = bias ? wld(bias, c) : 0.0f;
    for (uint32_t j = 0; j < taps; j++) {
        const int tau = (int)t - (int)(taps - 1) + (int)j;     // time relative to the step's first token
        const float x = tau >= 0 ? src[(size_t)tau * src_rs + c] : st[(size_t)(tau + (int)(taps - 1)) * C + c];
        y = fmaf(wld(w, (size_t)c * taps + j), x, y);
        // single-token steps: this thread alone touches the channel's carried inputs, so it also shifts them (input j moves to
        // row j - 1, which was read one trip earlier)
        if (advance && j > 0) st[(size_t)(j - 1) * C + c] = x;
    }
    if (act == 1) y = y * sigmoidf_(y);
    dst[(size_t)t * dst_rs + c] = y;
}
// state row r holds the input of time (first token of the NEXT step) - (taps - 1) + r; rows ascend, so shifting in place is safe
__global__ void k_conv_advance(float* __restrict__ state, const float* __restrict__ src, const float* __restrict__ ctl, uint32_t T, uint32_t C,
                               uint32_t taps, uint32_t src_rs) {
    pdl_enter();
    const uint32_t c = blockIdx.x * blockDim.x + threadIdx.x;
    if (c >= C) return;
    float* st = state + (size_t)ctl_word(ctl, ZG_CTL_SLOT) * (taps - 1) * C;
    for (uint32_t r = 0; r + 1 < taps; r++) {
        const int tau = (int)T - (int)(taps - 1) + (int)r;
        st[(size_t)r * C + c] = tau >= 0 ? src[(size_t)tau * src_rs + c] : st[(size_t)(r + T) * C + c];
    }
}

// ── DELTA_RULE ───────────────────────────────────────────────────────────────────────────────────────────────────
// Columns of the state evolve independently given the token's k, q, decay and beta, so a head is split by value columns
// over CTAs.  A thread keeps kDeltaRows consecutive key rows of one column in registers; the RS threads of a column sit in
// adjacent lanes and meet by shuffles.  The per-token vectors (unit k, scaled unit q, decay) of kDeltaTile tokens are
// prepared by the whole CTA at once, then the tokens are walked without further barriers.
constexpr int kDeltaRows = 16, kDeltaTile = 16, kDeltaThreads = 128;
// forms of the rule (op parameter n10): plain accumulation without unit vectors and correction (gated linear attention), the
// decay as a tempered sigmoid, a SiLU output gate, an output scale
constexpr uint32_t kDeltaPlain = 1, kDeltaSigmoidDecay = 2, kDeltaSiluGate = 4, kDeltaOutScale = 8;
// decay of one key channel from its logit z (the bias is already added): exp(-exp(A) softplus(z)), or sigmoid(z)^(1 / tau) =
// exp(-softplus(-z) / tau)
__device__ __forceinline__ float delta_decay(float z, float Ah, uint32_t form, float inv_tau) {
    return (form & kDeltaSigmoidDecay) ? expf(-softplusf_(-z) * inv_tau) : expf(-Ah * softplusf_(z));
}
template <typename WT>
__global__ void __launch_bounds__(kDeltaThreads) k_delta_rule(
    float* __restrict__ dst, const float* __restrict__ qkv, const float* __restrict__ betab, const float* __restrict__ ab, const WT* __restrict__ wts,
    float* __restrict__ state, const float* __restrict__ ctl, uint32_t T, uint32_t H, uint32_t G, uint32_t dim, uint32_t vdim, uint32_t RS,
    uint32_t q_off, uint32_t k_off, uint32_t v_off, uint32_t beta_off, uint32_t A_off, uint32_t dt_off, uint32_t qkv_rs, uint32_t beta_rs,
    uint32_t a_rs, float unit_eps, float q_scale, uint32_t form, float inv_tau, uint32_t dst_rs) {
    pdl_enter();
    extern __shared__ float sm[];
    const bool plain = form & kDeltaPlain;             // no unit vectors, no correction: S <- g S + k v^T
    const uint32_t dpad = RS * kDeltaRows;             // rows incl. padding (k = q = 0, decay = 1 there)
    float* sk = sm;                                    // [tile][dpad]
    float* sq = sk + kDeltaTile * dpad;
    float* sg = sq + kDeltaTile * dpad;
    float* sbeta = sg + kDeltaTile * dpad;             // [tile]
    const uint32_t h = blockIdx.y, kv = h / (H / G);
    const uint32_t cols_per_cta = kDeltaThreads / RS;
    const uint32_t r = threadIdx.x % RS, col = blockIdx.x * cols_per_cta + threadIdx.x / RS;
    const bool live = col < vdim;
    const uint32_t slot = (uint32_t)ctl_word(ctl, ZG_CTL_SLOT);
    float* S_g = state + (((size_t)slot * H + h) * dim) * vdim;
    float S[kDeltaRows];
#pragma unroll
    for (int i = 0; i < kDeltaRows; i++) {
        const uint32_t row = r * kDeltaRows + i;
        S[i] = (live && row < dim) ? S_g[(size_t)row * vdim + col] : 0.0f;
    }
    const float Ah = (form & kDeltaSigmoidDecay) ? 0.0f : expf(wld(wts, (size_t)A_off + h));
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    for (uint32_t t0 = 0; t0 < T; t0 += kDeltaTile) {
        const uint32_t nt = min((uint32_t)kDeltaTile, T - t0);
        __syncthreads();
        // prepare: warp w takes tokens w, w + 4, ...
        for (uint32_t tt = warp; tt < nt; tt += kDeltaThreads / 32) {
            const uint32_t t = t0 + tt;
            const float* qr = qkv + (size_t)t * qkv_rs + q_off + (size_t)kv * dim;
            const float* kr = qkv + (size_t)t * qkv_rs + k_off + (size_t)kv * dim;
            const float* ar = ab + (size_t)t * a_rs + (size_t)h * dim;
            float qn = q_scale, kn = 1.0f;
            if (!plain) {
                float qq = 0.0f, kk = 0.0f;
                for (uint32_t c = lane; c < dim; c += 32) { qq = fmaf(qr[c], qr[c], qq); kk = fmaf(kr[c], kr[c], kk); }
                qn = q_scale / sqrtf(warp_sum(qq) + unit_eps); kn = 1.0f / sqrtf(warp_sum(kk) + unit_eps);
            }
            for (uint32_t c = lane; c < dpad; c += 32) {
                const bool in = c < dim;
                sk[tt * dpad + c] = in ? kr[c] * kn : 0.0f;
                sq[tt * dpad + c] = in ? qr[c] * qn : 0.0f;
                sg[tt * dpad + c] = in ? delta_decay(ar[c] + wld(wts, (size_t)dt_off + (size_t)h * dim + c), Ah, form, inv_tau) : 1.0f;
            }
            if (lane == 0) sbeta[tt] = plain ? 1.0f : sigmoidf_(betab[(size_t)t * beta_rs + beta_off + h]);
        }
        float vt[kDeltaTile];                              // the tile's values of this column: independent loads, issued together
#pragma unroll
        for (int tt = 0; tt < kDeltaTile; tt++)
            vt[tt] = (live && (uint32_t)tt < nt) ? qkv[(size_t)(t0 + tt) * qkv_rs + v_off + (size_t)h * vdim + col] : 0.0f;
        __syncthreads();
#pragma unroll
        for (int tti = 0; tti < kDeltaTile; tti++) {
            const uint32_t tt = (uint32_t)tti;
            if (tt >= nt) break;
            const uint32_t t = t0 + tt;
            const float* k = sk + tt * dpad + r * kDeltaRows;
            const float* q = sq + tt * dpad + r * kDeltaRows;
            const float* g = sg + tt * dpad + r * kDeltaRows;
            const float v = vt[tti];
            float ks = 0.0f;
#pragma unroll
            for (int i = 0; i < kDeltaRows; i++) { S[i] *= g[i]; ks = fmaf(S[i], k[i], ks); }
            if (!plain) for (uint32_t o = 1; o < RS; o <<= 1) ks += __shfl_xor_sync(0xffffffffu, ks, o);
            const float u = plain ? v : sbeta[tt] * (v - ks);
            float os = 0.0f;
#pragma unroll
            for (int i = 0; i < kDeltaRows; i++) { S[i] = fmaf(k[i], u, S[i]); os = fmaf(S[i], q[i], os); }
            for (uint32_t o = 1; o < RS; o <<= 1) os += __shfl_xor_sync(0xffffffffu, os, o);
            if (live && r == 0) dst[(size_t)t * dst_rs + (size_t)h * vdim + col] = os;
        }
    }
#pragma unroll
    for (int i = 0; i < kDeltaRows; i++) {
        const uint32_t row = r * kDeltaRows + i;
        if (live && row < dim) S_g[(size_t)row * vdim + col] = S[i];
    }
}
// Prefill form of DELTA_RULE (kDeltaPrepMinTokens or more tokens): the per-token vectors are prepared for ALL tokens at
// once by k_delta_prepare (one warp per (token, head); the walk's critical path then holds no transcendental and no global
// read), into rows [unit k | scaled unit q | decay | beta, k . q, 0, 0] of 3 dpad + 4 floats laid out [head][token], so
// that a tile of tokens is one contiguous, 16-byte aligned block.  k_delta_walk streams those tiles into shared memory with
// cp.async, double buffered, and walks the tokens.  Per token a thread scales its rows by the decay and takes BOTH dot
// products, with k and with q, in the same pass; one shuffle round reduces them together.  The read-out after the write
// follows from  o = (g S)^T q + u (k . q), so the state update S <- g S + k u^T leaves the output's critical path.
// A thread's kWalkRows rows are groups of four consecutive rows, group c of slice r at row (c RS + r) 4: the RS slices
// of a column read consecutive float4s of a prepared vector (no bank conflict; the columns of a warp read the same words).
constexpr int kDeltaPrepMinTokens = 16;
// The walk keeps 16 rows per thread (four groups of four) and 128 threads per CTA.  (8 rows and 256 threads, two warps per
// scheduler, was measured slower: 388 against 354 us at 16 heads of 128 x 128 — the per-token dependency chain, which a
// fourth shuffle step lengthens, is what bounds the kernel, not the empty issue slots.)
constexpr int kWalkRows = 16, kWalkThreads = 128, kWalkMaxDim = 32 * kWalkRows;
static uint32_t delta_walk_slices(uint32_t dim) {
    uint32_t rs = 1;
    while (rs * kWalkRows < dim) rs <<= 1;
    return rs;
}
__device__ __forceinline__ uint32_t delta_row(uint32_t RS, uint32_t r, int i) { return (((uint32_t)i >> 2) * RS + r) * 4 + ((uint32_t)i & 3); }
template <typename WT>
__global__ void k_delta_prepare(float* __restrict__ prep, const float* __restrict__ qkv, const float* __restrict__ betab, const float* __restrict__ ab,
                                const WT* __restrict__ wts, uint32_t T, uint32_t H, uint32_t G, uint32_t dim, uint32_t dpad, uint32_t q_off,
                                uint32_t k_off, uint32_t beta_off, uint32_t A_off, uint32_t dt_off, uint32_t qkv_rs, uint32_t beta_rs, uint32_t a_rs,
                                float unit_eps, float q_scale, uint32_t form, float inv_tau) {
    pdl_enter();
    const bool plain = form & kDeltaPlain;
    const uint32_t w = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (w >= T * H) return;
    const uint32_t t = w / H, h = w % H, kv = h / (H / G);
    const float* qr = qkv + (size_t)t * qkv_rs + q_off + (size_t)kv * dim;
    const float* kr = qkv + (size_t)t * qkv_rs + k_off + (size_t)kv * dim;
    const float* ar = ab + (size_t)t * a_rs + (size_t)h * dim;
    float qq = 0.0f, kk = 0.0f, qk = 0.0f;
    for (uint32_t c = lane; c < dim; c += 32) { const float a = qr[c], b = kr[c]; qq = fmaf(a, a, qq); kk = fmaf(b, b, kk); qk = fmaf(a, b, qk); }
    const float qn = plain ? q_scale : q_scale / sqrtf(warp_sum(qq) + unit_eps), kn = plain ? 1.0f : 1.0f / sqrtf(warp_sum(kk) + unit_eps);
    qk = warp_sum(qk) * qn * kn;
    const float Ah = (form & kDeltaSigmoidDecay) ? 0.0f : expf(wld(wts, (size_t)A_off + h));
    float* row = prep + ((size_t)h * T + t) * (3 * dpad + 4);
    for (uint32_t c = lane; c < dpad; c += 32) {
        const bool in = c < dim;
        row[c] = in ? kr[c] * kn : 0.0f;
        row[dpad + c] = in ? qr[c] * qn : 0.0f;
        row[2 * dpad + c] = in ? delta_decay(ar[c] + wld(wts, (size_t)dt_off + (size_t)h * dim + c), Ah, form, inv_tau) : 1.0f;
    }
    if (lane < 4) row[3 * dpad + lane] = lane == 0 ? (plain ? 1.0f : sigmoidf_(betab[(size_t)t * beta_rs + beta_off + h])) : (lane == 1 ? qk : 0.0f);
}
__device__ __forceinline__ void cp_async16(float* smem_dst, const float* gmem_src) {
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16;" ::"r"((uint32_t)__cvta_generic_to_shared(smem_dst)), "l"(gmem_src) : "memory");
}
// PLAIN: the accumulation without correction (u = v), which needs no product with k and only one reduction per token
template <uint32_t RS, bool PLAIN>                     // row slices of a column: compile-time, so the shuffle steps unroll
__global__ void __launch_bounds__(kWalkThreads) k_delta_walk(float* __restrict__ dst, const float* __restrict__ qkv, const float* __restrict__ prep,
                                                               float* __restrict__ state, const float* __restrict__ ctl, uint32_t T, uint32_t H,
                                                               uint32_t dim, uint32_t vdim, uint32_t v_off, uint32_t qkv_rs, uint32_t dst_rs) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const uint32_t dpad = RS * kWalkRows, stride = 3 * dpad + 4, tile_elems = kDeltaTile * stride;
    const uint32_t h = blockIdx.y;
    const uint32_t cols_per_cta = kWalkThreads / RS;
    const uint32_t r = threadIdx.x % RS, col = blockIdx.x * cols_per_cta + threadIdx.x / RS;
    const bool live = col < vdim;
    const uint32_t slot = (uint32_t)ctl_word(ctl, ZG_CTL_SLOT);
    float* S_g = state + (((size_t)slot * H + h) * dim) * vdim;
    float S[kWalkRows];
#pragma unroll
    for (int i = 0; i < kWalkRows; i++) {
        const uint32_t row = delta_row(RS, r, i);
        S[i] = (live && row < dim) ? S_g[(size_t)row * vdim + col] : 0.0f;
    }
    const float* P = prep + (size_t)h * T * stride;
    const float* vbase = qkv + v_off + (size_t)h * vdim + col;
    auto stage = [&](uint32_t t0, float* buf) {       // rows of tokens [t0, min(t0 + tile, T)): one contiguous block
        const uint32_t n4 = min((uint32_t)kDeltaTile, T - t0) * stride / 4;
        const float* src = P + (size_t)t0 * stride;
        for (uint32_t i = threadIdx.x; i < n4; i += kWalkThreads) cp_async16(buf + 4 * i, src + 4 * i);
        asm volatile("cp.async.commit_group;" ::: "memory");
    };
    stage(0, sm);
    float vt[kDeltaTile];
#pragma unroll
    for (int tt = 0; tt < kDeltaTile; tt++) vt[tt] = (live && (uint32_t)tt < T) ? vbase[(size_t)tt * qkv_rs] : 0.0f;
    uint32_t cur = 0;
    for (uint32_t t0 = 0; t0 < T; t0 += kDeltaTile, cur ^= 1) {
        const uint32_t nt = min((uint32_t)kDeltaTile, T - t0);
        const bool more = t0 + kDeltaTile < T;
        if (more) stage(t0 + kDeltaTile, sm + (cur ^ 1) * tile_elems);   // its last readers passed the barrier that ended the tile before
        float vn[kDeltaTile];                                             // the next tile's values of this column, in flight during the walk
#pragma unroll
        for (int tt = 0; tt < kDeltaTile; tt++)
            vn[tt] = (live && more && t0 + kDeltaTile + tt < T) ? vbase[(size_t)(t0 + kDeltaTile + tt) * qkv_rs] : 0.0f;
        if (more) asm volatile("cp.async.wait_group 1;" ::: "memory"); else asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        const float* tile = sm + cur * tile_elems;
        auto token = [&](int tti, float v) {
            const float* row = tile + tti * stride;
            const float beta = row[3 * dpad], kq = row[3 * dpad + 1];   // read with the vectors, before the shuffles
            float4 k4[kWalkRows / 4], g4[kWalkRows / 4];
            float ks0 = 0.0f, ks1 = 0.0f, qs0 = 0.0f, qs1 = 0.0f;
#pragma unroll
            for (int c = 0; c < kWalkRows / 4; c++) {
                const uint32_t at = (c * RS + r) * 4;
                k4[c] = *reinterpret_cast<const float4*>(row + at);
                const float4 q4 = *reinterpret_cast<const float4*>(row + dpad + at);
                g4[c] = *reinterpret_cast<const float4*>(row + 2 * dpad + at);
                S[4 * c + 0] *= g4[c].x; S[4 * c + 1] *= g4[c].y; S[4 * c + 2] *= g4[c].z; S[4 * c + 3] *= g4[c].w;
                if (!PLAIN) {
                    ks0 = fmaf(S[4 * c + 0], k4[c].x, ks0); ks1 = fmaf(S[4 * c + 1], k4[c].y, ks1);
                    ks0 = fmaf(S[4 * c + 2], k4[c].z, ks0); ks1 = fmaf(S[4 * c + 3], k4[c].w, ks1);
                }
                qs0 = fmaf(S[4 * c + 0], q4.x, qs0); qs1 = fmaf(S[4 * c + 1], q4.y, qs1);
                qs0 = fmaf(S[4 * c + 2], q4.z, qs0); qs1 = fmaf(S[4 * c + 3], q4.w, qs1);
            }
            float ks = ks0 + ks1, qs = qs0 + qs1;
#pragma unroll
            for (uint32_t o = 1; o < RS; o <<= 1) { if (!PLAIN) ks += __shfl_xor_sync(0xffffffffu, ks, o); qs += __shfl_xor_sync(0xffffffffu, qs, o); }
            const float u = PLAIN ? v : beta * (v - ks);
#pragma unroll
            for (int c = 0; c < kWalkRows / 4; c++) {
                S[4 * c + 0] = fmaf(k4[c].x, u, S[4 * c + 0]); S[4 * c + 1] = fmaf(k4[c].y, u, S[4 * c + 1]);
                S[4 * c + 2] = fmaf(k4[c].z, u, S[4 * c + 2]); S[4 * c + 3] = fmaf(k4[c].w, u, S[4 * c + 3]);
            }
            if (live && r == 0) dst[(size_t)(t0 + tti) * dst_rs + (size_t)h * vdim + col] = fmaf(u, kq, qs);
        };
        if (nt == (uint32_t)kDeltaTile) {                  // a full tile: straight-line code, nothing between the tokens
#pragma unroll
            for (int tti = 0; tti < kDeltaTile; tti++) token(tti, vt[tti]);
        } else {
#pragma unroll
            for (int tti = 0; tti < kDeltaTile; tti++) {
                if ((uint32_t)tti >= nt) break;
                token(tti, vt[tti]);
            }
        }
#pragma unroll
        for (int tt = 0; tt < kDeltaTile; tt++) vt[tt] = vn[tt];
        __syncthreads();                                   // everyone is done with this buffer: the next iteration refills it
    }
#pragma unroll
    for (int i = 0; i < kWalkRows; i++) {
        const uint32_t row = delta_row(RS, r, i);
        if (live && row < dim) S_g[(size_t)row * vdim + col] = S[i];
    }
}
// o / rms(o) * norm_w * sigmoid(gate) (or silu(gate)) * out_scale, one warp per (token, head), in place
template <typename WT>
__global__ void k_delta_out(float* __restrict__ dst, const float* __restrict__ gate, const WT* __restrict__ wts, uint32_t TH, uint32_t H,
                            uint32_t vdim, uint32_t gate_rs, uint32_t nw_off, float eps, uint32_t dst_rs, uint32_t silu_gate, float out_scale) {
    pdl_enter();
    const uint32_t item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= TH) return;
    const uint32_t t = item / H, h = item % H;
    float* o = dst + (size_t)t * dst_rs + (size_t)h * vdim;
    const float* g = gate + (size_t)t * gate_rs + (size_t)h * vdim;
    float q = 0.0f;
    for (uint32_t c = lane; c < vdim; c += 32) q = fmaf(o[c], o[c], q);
    const float inv = out_scale / sqrtf(warp_sum(q) / (float)vdim + eps);
    for (uint32_t c = lane; c < vdim; c += 32) o[c] = o[c] * inv * wld(wts, (size_t)nw_off + c) * (silu_gate ? g[c] * sigmoidf_(g[c]) : sigmoidf_(g[c]));
}

// ── ROUTE: one warp per token ────────────────────────────────────────────────────────────────────────────────────
template <typename WT>
__global__ void k_route(float* __restrict__ dst, const float* __restrict__ logits, const WT* __restrict__ corr, uint32_t T, uint32_t NE, uint32_t top,
                        uint32_t logits_rs, uint32_t mode, uint32_t groups, uint32_t keep) {
    pdl_enter();
    extern __shared__ float sm[];                      // [warps][NE + groups] choice scores, group scores
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31;
    const uint32_t t = blockIdx.x * (blockDim.x >> 5) + warp;
    if (t >= T) return;
    const float* z = logits + (size_t)t * logits_rs;
    float* ch = sm + warp * (NE + groups);
    float mx = -INFINITY, inv = 0.0f;
    if (mode == 0) {
        for (uint32_t e = lane; e < NE; e += 32) mx = fmaxf(mx, z[e]);
        mx = warp_max(mx);
        float sum = 0.0f;
        for (uint32_t e = lane; e < NE; e += 32) sum += expf(z[e] - mx);
        inv = 1.0f / warp_sum(sum);
        for (uint32_t e = lane; e < NE; e += 32) ch[e] = expf(z[e] - mx) * inv + wld(corr, e);
    } else if (mode == 1) {
        for (uint32_t e = lane; e < NE; e += 32) ch[e] = z[e] + wld(corr, e);   // biased logits choose AND weigh
    } else {
        for (uint32_t e = lane; e < NE; e += 32) ch[e] = sigmoidf_(z[e]) + wld(corr, e);
        if (groups > 1) {                              // only outputs of the `keep` best groups stay eligible
            float* gs = ch + NE;
            const uint32_t per = NE / groups;
            __syncwarp();
            for (uint32_t g = lane; g < groups; g += 32) {   // a group scores the sum of its two largest choice scores
                float a = -INFINITY, b = -INFINITY;
                for (uint32_t e = g * per; e < (g + 1) * per; e++) {
                    const float v = ch[e];
                    if (v > a) { b = a; a = v; } else if (v > b) b = v;
                }
                gs[g] = per > 1 ? a + b : a;
            }
            __syncwarp();
            uint32_t kept_mine = 0;                    // bit i: group lane + 32 i is kept (groups <= 1024)
            for (uint32_t c = 0; c < keep; c++) {
                float best = -INFINITY; uint32_t bi = 0xFFFFFFFFu;
                for (uint32_t g = lane; g < groups; g += 32) if (!((kept_mine >> (g / 32)) & 1u) && (gs[g] > best || bi == 0xFFFFFFFFu)) { best = gs[g]; bi = g; }
                for (int o = 16; o > 0; o >>= 1) {
                    const float ob = __shfl_xor_sync(0xffffffffu, best, o);
                    const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
                    if (oi != 0xFFFFFFFFu && (bi == 0xFFFFFFFFu || ob > best || (ob == best && oi < bi))) { best = ob; bi = oi; }
                }
                if (bi != 0xFFFFFFFFu && bi % 32 == lane) kept_mine |= 1u << (bi / 32);
            }
            for (uint32_t g = lane; g < groups; g += 32)
                if (!((kept_mine >> (g / 32)) & 1u))
                    for (uint32_t e = g * per; e < (g + 1) * per; e++) ch[e] = -INFINITY;
        }
    }
    __syncwarp();
    float first = 0.0f, chosen_sum = 0.0f;             // mode 1 (lane 0): the largest chosen logit and the sum of exp(z - first)
    for (uint32_t c = 0; c < top; c++) {
        float best = -INFINITY; uint32_t bi = 0xFFFFFFFFu;
        for (uint32_t e = lane; e < NE; e += 32) if (ch[e] > best) { best = ch[e]; bi = e; }
        for (int o = 16; o > 0; o >>= 1) {
            const float ob = __shfl_xor_sync(0xffffffffu, best, o);
            const uint32_t oi = __shfl_xor_sync(0xffffffffu, bi, o);
            if (ob > best || (ob == best && oi < bi)) { best = ob; bi = oi; }
        }
        if (lane == 0) {
            float* out = dst + ((size_t)t * top + c) * 2;
            reinterpret_cast<int*>(out)[0] = (int)bi;
            if (mode == 0) out[1] = bi < NE ? expf(z[bi] - mx) * inv : 0.0f;
            else if (mode == 2) { out[1] = bi < NE ? sigmoidf_(z[bi]) : 0.0f; chosen_sum += out[1]; }
            else {
                if (c == 0) first = best;
                out[1] = bi < NE ? expf(best - first) : 0.0f;
                chosen_sum += out[1];
            }
            if (bi < NE) ch[bi] = -INFINITY;
        }
        __syncwarp();
    }
    if (mode != 0 && lane == 0) {
        const float norm = 1.0f / (mode == 2 ? chosen_sum + 1e-20f : chosen_sum);
        for (uint32_t c = 0; c < top; c++) dst[((size_t)t * top + c) * 2 + 1] *= norm;
    }
}

// dot of one weight row with an f32 vector by a whole warp (every lane gets the sum); 16-byte weight loads when aligned,
// four of them in flight per lane (a row is streamed once, so what hides HBM latency is the number of independent loads)
template <typename WT>
__device__ __forceinline__ float fma_vec4(const float* wv, const float* __restrict__ x, float acc) {
    constexpr int V = WVec<WT>::n;
#pragma unroll
    for (int i = 0; i < V / 4; i++) {
        const float4 xv = *reinterpret_cast<const float4*>(x + 4 * i);
        acc = fmaf(xv.x, wv[4 * i], fmaf(xv.y, wv[4 * i + 1], fmaf(xv.z, wv[4 * i + 2], fmaf(xv.w, wv[4 * i + 3], acc))));
    }
    return acc;
}
template <typename WT>
__device__ __forceinline__ float warp_dot(const WT* __restrict__ w, const float* __restrict__ x, uint32_t K, uint32_t lane) {
    constexpr int V = WVec<WT>::n;
    float acc = 0.0f;
    if (K % V == 0 && (reinterpret_cast<size_t>(w) & 15) == 0 && (reinterpret_cast<size_t>(x) & 15) == 0) {
        float a1 = 0.0f, a2 = 0.0f, a3 = 0.0f;
        uint32_t k = lane * V;
        for (; k + 96 * V < K; k += 128 * V) {
            float w0[V], w1[V], w2[V], w3[V];
            wld_vec<WT>(w + k, w0); wld_vec<WT>(w + k + 32 * V, w1); wld_vec<WT>(w + k + 64 * V, w2); wld_vec<WT>(w + k + 96 * V, w3);
            acc = fma_vec4<WT>(w0, x + k, acc); a1 = fma_vec4<WT>(w1, x + k + 32 * V, a1);
            a2 = fma_vec4<WT>(w2, x + k + 64 * V, a2); a3 = fma_vec4<WT>(w3, x + k + 96 * V, a3);
        }
        for (; k < K; k += 32 * V) {
            float w0[V];
            wld_vec<WT>(w + k, w0);
            acc = fma_vec4<WT>(w0, x + k, acc);
        }
        acc = (acc + a1) + (a2 + a3);
    } else {
        for (uint32_t k = lane; k < K; k += 32) acc = fmaf(x[k], wld(w, k), acc);
    }
    return warp_sum(acc);
}
// two rows against the same vector, their loads interleaved (the gate and up rows of an expert)
template <typename WT>
__device__ __forceinline__ void warp_dot2(const WT* __restrict__ wa, const WT* __restrict__ wb, const float* __restrict__ x, uint32_t K, uint32_t lane,
                                          float& ra, float& rb) {
    constexpr int V = WVec<WT>::n;
    if (K % V == 0 && (reinterpret_cast<size_t>(wa) & 15) == 0 && (reinterpret_cast<size_t>(wb) & 15) == 0 && (reinterpret_cast<size_t>(x) & 15) == 0) {
        float a0 = 0.0f, a1 = 0.0f, b0 = 0.0f, b1 = 0.0f;
        uint32_t k = lane * V;
        for (; k + 32 * V < K; k += 64 * V) {
            float p0[V], p1[V], q0[V], q1[V];
            wld_vec<WT>(wa + k, p0); wld_vec<WT>(wb + k, q0); wld_vec<WT>(wa + k + 32 * V, p1); wld_vec<WT>(wb + k + 32 * V, q1);
            a0 = fma_vec4<WT>(p0, x + k, a0); b0 = fma_vec4<WT>(q0, x + k, b0);
            a1 = fma_vec4<WT>(p1, x + k + 32 * V, a1); b1 = fma_vec4<WT>(q1, x + k + 32 * V, b1);
        }
        for (; k < K; k += 32 * V) {
            float p0[V], q0[V];
            wld_vec<WT>(wa + k, p0); wld_vec<WT>(wb + k, q0);
            a0 = fma_vec4<WT>(p0, x + k, a0); b0 = fma_vec4<WT>(q0, x + k, b0);
        }
        ra = warp_sum(a0 + a1); rb = warp_sum(b0 + b1);
    } else {
        ra = warp_dot(wa, x, K, lane); rb = warp_dot(wb, x, K, lane);
    }
}

// ── MOE_FFN, token-wise form: every (token, choice) pair streams the rows of its expert (decode and short steps) ────────
template <typename WT>
__global__ void k_moe_up(float* __restrict__ y, const float* __restrict__ src, const float* __restrict__ route, const WT* __restrict__ wg,
                         const WT* __restrict__ wu, uint32_t D, uint32_t ff, uint32_t E, uint32_t top, float limit, float alpha, float uoff, uint32_t stage) {
    pdl_enter();
    const uint32_t pair = blockIdx.y;                  // token * top + choice
    const uint32_t f = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    const uint32_t e = (uint32_t)reinterpret_cast<const int*>(route)[2 * (size_t)pair];
    if (e >= E) return;                                // identity experts have no weights (uniform over the CTA)
    extern __shared__ __align__(16) float xsh[];       // the token's input, staged once per CTA when it fits
    const float* x = src + (size_t)(pair / top) * D;
    if (stage) {
        for (uint32_t c = threadIdx.x; c < D; c += blockDim.x) xsh[c] = x[c];
        __syncthreads();
        x = xsh;
    }
    if (f >= ff) return;
    const size_t row = ((size_t)e * ff + f) * D;
    float g, u;
    warp_dot2(wg + row, wu + row, x, D, lane, g, u);
    g = fminf(g, limit);
    u = fminf(fmaxf(u, -limit), limit);
    if (lane == 0) y[(size_t)pair * ff + f] = g * sigmoidf_(alpha * g) * (u + uoff);
}
template <typename WT>
__global__ void k_moe_down(float* __restrict__ dst, const float* __restrict__ src, const float* __restrict__ y, const float* __restrict__ route,
                           const WT* __restrict__ wd, uint32_t D, uint32_t ff, uint32_t E, uint32_t top) {
    pdl_enter();
    const uint32_t t = blockIdx.y;
    const uint32_t d = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (d >= D) return;
    float acc = 0.0f;
    for (uint32_t c = 0; c < top; c++) {               // fixed order: the result does not depend on the launch shape
        const size_t pair = (size_t)t * top + c;
        const uint32_t e = (uint32_t)reinterpret_cast<const int*>(route)[2 * pair];
        const float w = route[2 * pair + 1];
        const float v = e < E ? warp_dot(wd + ((size_t)e * D + d) * ff, y + pair * ff, ff, lane) : src[(size_t)t * D + d];
        acc = fmaf(w, v, acc);
    }
    if (lane == 0) dst[(size_t)t * D + d] = acc;
}

// ── MOE_FFN, grouped form (prefill on bfloat16 sessions): the step's (token, choice) pairs are sorted by expert into whole
// 128-row tiles, the rows are gathered as bf16, and every expert's gate / up / down products run as tiles of ONE grouped
// tensor-core matmul each (dense_gemm.cu), so an expert's weights are read once per 128 rows instead of once per token ──
struct MoeLayout {          // offsets in f32 slots inside the op's scratch operand
    uint32_t R, Dp, Fp;     // rows incl. per-expert padding, padded widths of the bf16 copies
    size_t tile_group, row_pair, pos_of_pair, xs, g, u, yb, z, total;
};
__host__ __device__ inline size_t up4(size_t n) { return (n + 3) & ~(size_t)3; }
MoeLayout moe_layout(uint32_t T, uint32_t D, uint32_t ff, uint32_t E, uint32_t top) {
    MoeLayout L;
    L.R = (T * top + 127) / 128 * 128 + E * 128;
    L.Dp = (D + 63) / 64 * 64; L.Fp = (ff + 63) / 64 * 64;
    size_t o = 0;
    L.tile_group = o; o = up4(o + L.R / 128);
    L.row_pair = o; o = up4(o + L.R);
    L.pos_of_pair = o; o = up4(o + (size_t)T * top);
    L.xs = o; o = up4(o + (size_t)L.R * L.Dp / 2);
    L.g = o; o = up4(o + (size_t)L.R * ff);
    L.u = o; o = up4(o + (size_t)L.R * ff);
    L.yb = o; o = up4(o + (size_t)L.R * L.Fp / 2);
    L.z = o; o = up4(o + (size_t)L.R * D);
    L.total = o;
    return L;
}
constexpr uint32_t kMoeMaxExperts = 1024;
__global__ void __launch_bounds__(1024) k_moe_sort(const float* __restrict__ route, int* __restrict__ tile_group, int* __restrict__ row_pair,
                                                   int* __restrict__ pos_of_pair, uint32_t pairs, uint32_t E, uint32_t R) {
    __shared__ int cnt[kMoeMaxExperts], off[kMoeMaxExperts + 1];
    for (uint32_t e = threadIdx.x; e < E; e += blockDim.x) cnt[e] = 0;
    for (uint32_t r = threadIdx.x; r < R; r += blockDim.x) row_pair[r] = -1;
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < pairs; i += blockDim.x) {
        const uint32_t e = (uint32_t)reinterpret_cast<const int*>(route)[2 * (size_t)i];
        if (e < E) atomicAdd(&cnt[e], 1);
    }
    __syncthreads();
    if (threadIdx.x == 0) {
        int o = 0;
        for (uint32_t e = 0; e < E; e++) {
            off[e] = o;
            const int tiles = (cnt[e] + 127) / 128;
            for (int t = 0; t < tiles; t++) tile_group[o / 128 + t] = (int)e;
            o += tiles * 128;
            cnt[e] = 0;                                  // becomes the expert's fill cursor
        }
        for (uint32_t t = (uint32_t)o / 128; t < R / 128; t++) tile_group[t] = -1;
    }
    __syncthreads();
    for (uint32_t i = threadIdx.x; i < pairs; i += blockDim.x) {
        const uint32_t e = (uint32_t)reinterpret_cast<const int*>(route)[2 * (size_t)i];
        int pos = -1;
        if (e < E) { pos = off[e] + atomicAdd(&cnt[e], 1); row_pair[pos] = (int)i; }
        pos_of_pair[i] = pos;                            // which row a pair landed in does not change its result
    }
}
__global__ void k_moe_gather(uint32_t* __restrict__ xs, const float* __restrict__ src, const int* __restrict__ row_pair, uint32_t D, uint32_t dp2,
                             uint32_t top) {
    const uint32_t r = blockIdx.x;
    const int pair = row_pair[r];
    const float* x = pair >= 0 ? src + (size_t)((uint32_t)pair / top) * D : nullptr;
    for (uint32_t k2 = threadIdx.x; k2 < dp2; k2 += blockDim.x) {
        const uint32_t k = 2 * k2;
        const float a = (x && k < D) ? x[k] : 0.0f, b = (x && k + 1 < D) ? x[k + 1] : 0.0f;
        uint32_t v;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(v) : "f"(b), "f"(a));
        xs[(size_t)r * dp2 + k2] = v;
    }
}
__global__ void k_moe_act(uint32_t* __restrict__ yb, const float* __restrict__ g, const float* __restrict__ u, const int* __restrict__ row_pair,
                          uint32_t ff, uint32_t fp2, float limit, float alpha, float uoff) {
    const uint32_t r = blockIdx.x;
    const bool live = row_pair[r] >= 0;
    for (uint32_t f2 = threadIdx.x; f2 < fp2; f2 += blockDim.x) {
        float y[2] = {0.0f, 0.0f};
        for (int i = 0; i < 2; i++) {
            const uint32_t f = 2 * f2 + i;
            if (live && f < ff) {
                const float gv = fminf(g[(size_t)r * ff + f], limit), uv = fminf(fmaxf(u[(size_t)r * ff + f], -limit), limit);
                y[i] = gv * sigmoidf_(alpha * gv) * (uv + uoff);
            }
        }
        uint32_t v;
        asm("cvt.rn.bf16x2.f32 %0, %1, %2;" : "=r"(v) : "f"(y[1]), "f"(y[0]));
        yb[(size_t)r * fp2 + f2] = v;
    }
}
__global__ void k_moe_combine(float* __restrict__ dst, const float* __restrict__ src, const float* __restrict__ z, const float* __restrict__ route,
                              const int* __restrict__ pos_of_pair, uint32_t D, uint32_t top) {
    const uint32_t t = blockIdx.x;
    for (uint32_t d = threadIdx.x; d < D; d += blockDim.x) {
        float acc = 0.0f;
        for (uint32_t c = 0; c < top; c++) {
            const size_t pair = (size_t)t * top + c;
            const int pos = pos_of_pair[pair];
            acc = fmaf(route[2 * pair + 1], pos >= 0 ? z[(size_t)pos * D + d] : src[(size_t)t * D + d], acc);
        }
        dst[(size_t)t * D + d] = acc;
    }
}

}  // namespace

static bool dense_gemm_enabled() {
    static const bool enabled = [] { const char* e = getenv("ZG_DENSE_GEMM"); return !(e && e[0] == '0'); }();
    return enabled;
}
// MOE_FFN on bfloat16 weights with enough (token, choice) pairs to fill tiles runs grouped on the tensor cores
static bool moe_grouped(const ZgSeqOp& s, float* const* bufs) {
    const uint32_t T = s.n[0], D = s.n[1], ff = s.n[2], E = s.n[3], top = s.n[4];
    if (!dense_gemm_enabled() || s.n[5] != ZG_W_BF16 || !E || E > kMoeMaxExperts || T * top <= 16 || D < 64 || ff < 64 || D % 8 || ff % 8) return false;
    if (!bufs) return true;
    for (int i = 0; i < 3; i++) if (reinterpret_cast<uintptr_t>(wptr<bf16>(bufs, s.buf[3], s.off[i])) & 15) return false;
    return true;
}
// f32 slots the op's own scratch operand (MOE_FFN buf[4]) must have; 0 for ops without one
size_t zg_seq_op_operand_scratch(const ZgOp& op) {
    if (op.tag != ZG_OP_MOE_FFN) return 0;
    const ZgSeqOp& s = op.u.seq;
    size_t n = (size_t)s.n[0] * s.n[4] * s.n[2];
    if (moe_grouped(s, nullptr)) { const size_t g = moe_layout(s.n[0], s.n[1], s.n[2], s.n[3], s.n[4]).total; if (g > n) n = g; }
    return n ? n : 1;
}
extern "C" __attribute__((visibility("default"))) size_t zg_cuda_seq_scratch_elems(const ZgOp* op) { return op ? zg_seq_op_operand_scratch(*op) : 0; }

uint32_t zg_delta_row_slices(uint32_t dim) {
    uint32_t rs = 1;
    while (rs * kDeltaRows < dim) rs <<= 1;
    return rs;
}

// Static checks of a sequence op against the program's buffer sizes (f32 slots): shapes, strides and every extent.
bool zg_seq_op_valid(const ZgOp& op, const size_t* elems, size_t n_bufs, char* why, size_t why_n) {
    if (op.tag >= ZG_OP_SSM_SCAN) return zg_rec_op_valid(op, elems, n_bufs, why, why_n);
    if (op.tag >= ZG_OP_TOKEN_SHIFT) return zg_mix_op_valid(op, elems, n_bufs, why, why_n);
    const ZgSeqOp& s = op.u.seq;
    auto fail = [&](const char* m) { snprintf(why, why_n, "%s", m); return false; };
    auto have = [&](int i) { return s.buf[i] != ZG_NO_BUF && s.buf[i] < n_bufs; };
    auto fits = [&](int i, size_t off, size_t n) { return have(i) && off + n <= elems[s.buf[i]]; };
    const uint32_t wdt_of[] = {s.n[2], s.n[5], s.n[3], 0, s.n[6], s.n[9], s.n[4], s.n[5]};
    const uint32_t wdt = wdt_of[op.tag - ZG_OP_EMBED];
    if (wdt > ZG_W_BF16) return fail("unknown weight type");
    auto wfits = [&](int i, size_t off, size_t n) { return have(i) && (wdt == ZG_W_BF16 ? (off + n + 1) / 2 : off + n) <= elems[s.buf[i]]; };
    switch (op.tag) {
        case ZG_OP_EMBED: {
            const size_t T = s.n[0], D = s.n[1];
            if (!fits(0, 0, T * D) || !fits(1, ZG_CTL_IDS, T) || !have(2)) return fail("embed: extent");
            return true;
        }
        case ZG_OP_LINEAR: {
            const size_t M = s.n[0], N = s.n[1], K = s.n[2], srs = s.n[3], drs = s.n[4];
            if (!M || !N || !K || srs < K || drs < N) return fail("linear: shape");
            if (!fits(0, s.off[3], (M - 1) * drs + N) || !fits(1, s.off[2], (M - 1) * srs + K) || !wfits(2, s.off[0], N * K)) return fail("linear: extent");
            if (s.buf[3] != ZG_NO_BUF && !wfits(3, s.off[1], N)) return fail("linear: bias extent");
            if (s.buf[0] == s.buf[1]) return fail("linear: in place");
            if (s.n[6] > 5 || (s.n[6] == 5 && !(s.f[0] > 0.0f))) return fail("linear: activation");
            if (s.n[7] && (s.n[7] < s.off[2] + (M - 1) * srs + K || !fits(4, 0, ZG_CTL_IDS))) return fail("linear: source slots");
            return true;
        }
        case ZG_OP_NORM: {
            const size_t n = (size_t)s.n[0] * s.n[1];
            if (!n || s.n[2] > 31 || (s.n[2] & 24u) == 24u) return fail("norm: shape");
            const size_t w_need = (s.n[2] & 8u) ? 2 * (size_t)s.n[1] + 1 : s.n[1];      // Dynamic Tanh: weight, bias and alpha
            if (!fits(0, s.off[3], n) || !fits(1, 0, n) || (!(s.n[2] & 16u) && !wfits(2, s.off[0], w_need))) return fail("norm: extent");
            if (s.n[7]) {      // a second source, normed like the first with its own weight (off 2 of w's arena) and added to it
                if (s.n[7] > 1 || (s.n[2] & 24u) || s.n[5] || !fits(6, 0, n) || !wfits(2, s.off[2], s.n[1]) || s.buf[6] == s.buf[0] || (s.buf[4] != ZG_NO_BUF && s.buf[6] == s.buf[4]))
                    return fail("norm: second source");
            } else if (((s.n[2] | (s.buf[4] != ZG_NO_BUF && !s.n[5] ? s.n[4] : 0u)) & 24u) && (s.n[5] || s.buf[6] != ZG_NO_BUF))
                return fail("norm: kinds without statistics take no averaged source and no token shift");
            if (s.n[5]) {      // averaged source
                if (s.n[6] < n || !fits(1, 0, (size_t)(s.n[5] - 1) * s.n[6] + n) || !wfits(2, s.off[4], s.n[5]) || s.buf[3] != ZG_NO_BUF || !fits(4, 0, n) || s.buf[4] == s.buf[0] ||
                    s.buf[4] == s.buf[1])
                    return fail("norm: averaged source");
                if (s.buf[6] != ZG_NO_BUF && (s.n[0] != 1 || !have(6) || elems[s.buf[6]] < s.n[1] || !wfits(2, s.off[2], s.n[1]) || !fits(7, 0, ZG_CTL_IDS))) return fail("norm: fused token shift (single-row steps)");
                return true;
            }
            if (s.buf[3] != ZG_NO_BUF && !fits(3, 0, n)) return fail("norm: residual extent");
            if (s.buf[4] != ZG_NO_BUF && (s.n[4] > 31 || (s.n[4] & 24u) == 24u || !fits(4, 0, n) || (!(s.n[4] & 16u) && !wfits(5, s.off[1], (s.n[4] & 8u) ? 2 * (size_t)s.n[1] + 1 : s.n[1])) || s.buf[4] == s.buf[0] || s.buf[4] == s.buf[1] || s.buf[4] == s.buf[3]))
                return fail("norm: chained norm");
            if (!s.n[7] && s.buf[6] != ZG_NO_BUF && (s.n[0] != 1 || !have(6) || elems[s.buf[6]] < s.n[1] || !wfits(s.buf[4] != ZG_NO_BUF ? 5 : 2, s.off[2], s.n[1]) || !fits(7, 0, ZG_CTL_IDS)))
                return fail("norm: fused token shift (single-row steps)");
            return true;
        }
        case ZG_OP_WINDOW_ATTENTION: {
            const size_t T = s.n[0], H = s.n[1], G = s.n[2], dim = s.n[3], rs = s.n[4], win = s.n[5], R = s.n[6];
            if (!T || !H || !G || H % G || !dim || dim > kAttnMaxDim || !win || R < win - 1 + T) return fail("window_attention: shape");
            if (s.off[0] + H * dim > rs || s.off[1] + G * dim > rs || s.off[2] + H * dim > rs) return fail("window_attention: columns");
            if (!fits(0, 0, T * H * dim) || !fits(1, 0, T * rs) || !have(2) || elems[s.buf[2]] < R * G * dim || !fits(3, 0, win * H) || !fits(4, 0, ZG_CTL_IDS))
                return fail("window_attention: extent");
            return true;
        }
        case ZG_OP_CAUSAL_CONV: {
            const size_t T = s.n[0], C = s.n[1], taps = s.n[2], srs = s.n[3], drs = s.n[4];
            if (!T || !C || taps < 1 || srs < C || drs < C || s.n[5] > 1) return fail("causal_conv: shape");
            if (!fits(0, s.off[2], (T - 1) * drs + C) || !fits(1, s.off[1], (T - 1) * srs + C) || !wfits(2, s.off[0], C * taps) || !have(3) || !fits(4, 0, ZG_CTL_IDS))
                return fail("causal_conv: extent");
            if (taps > 1 && elems[s.buf[3]] < (taps - 1) * C) return fail("causal_conv: state size");
            if (s.n[7] > 1 || (s.n[7] && !wfits(2, s.off[3], C))) return fail("causal_conv: bias");
            if (s.buf[0] == s.buf[1]) return fail("causal_conv: in place");
            return true;
        }
        case ZG_OP_DELTA_RULE: {
            const size_t T = s.n[0], H = s.n[1], G = s.n[2], dim = s.n[3], vdim = s.n[4];
            const size_t form = s.n[10], drs = s.n[11] ? s.n[11] : H * vdim;
            if (!T || !H || !G || H % G || !dim || !vdim || zg_delta_row_slices((uint32_t)dim) > 32 || form > 15) return fail("delta_rule: shape");
            if (s.n[12] + H * vdim > drs || ((form & 2) && !(s.f[3] > 0.0f))) return fail("delta_rule: form");
            if (s.off[0] + G * dim > s.n[5] || s.off[1] + G * dim > s.n[5] || s.off[2] + H * vdim > s.n[5] || (!(form & 1) && s.off[3] + H > s.n[6]) || H * dim > s.n[7] || s.off[7] + H * vdim > s.n[8])
                return fail("delta_rule: columns");
            if (!fits(0, 0, (T - 1) * drs + s.n[12] + H * vdim) || !fits(1, 0, T * s.n[5]) || (!(form & 1) && !fits(2, 0, T * s.n[6])) || !fits(3, 0, T * s.n[7]) || !fits(4, 0, T * s.n[8]) ||
                (!(form & 2) && !wfits(5, s.off[4], H)) || !wfits(5, s.off[5], H * dim) || !wfits(5, s.off[6], vdim) || !have(6) || elems[s.buf[6]] < H * dim * vdim || !fits(7, 0, ZG_CTL_IDS))
                return fail("delta_rule: extent");
            return true;
        }
        case ZG_OP_ROUTE: {
            const size_t T = s.n[0], NE = s.n[1], top = s.n[2], rs = s.n[3];
            if (!T || !NE || !top || top > NE || rs < NE || NE > 4096 || s.n[5] > 2) return fail("route: shape");
            if (s.n[5] == 2 && s.n[6] > 1 && (NE % s.n[6] || s.n[6] > 1024 || !s.n[7] || s.n[7] > s.n[6] || (size_t)s.n[7] * (NE / s.n[6]) < top)) return fail("route: groups");
            if (!fits(0, 0, T * top * 2) || !fits(1, s.off[1], (T - 1) * rs + NE) || !wfits(2, s.off[0], NE)) return fail("route: extent");
            return true;
        }
        case ZG_OP_MOE_FFN: {
            const size_t T = s.n[0], D = s.n[1], ff = s.n[2], E = s.n[3], top = s.n[4];
            if (!T || !D || !top) return fail("moe_ffn: shape");
            if (!fits(0, 0, T * D) || !fits(1, 0, T * D) || !fits(2, 0, T * top * 2) || !fits(4, 0, zg_seq_op_operand_scratch(op)) ||
                (E && (!wfits(3, s.off[0], E * ff * D) || !wfits(3, s.off[1], E * ff * D) || !wfits(3, s.off[2], E * ff * D))))
                return fail("moe_ffn: extent");
            if (s.buf[0] == s.buf[1]) return fail("moe_ffn: in place");
            return true;
        }
        default: return fail("not a sequence op");
    }
}

// which of buf[0..8) an op writes (bit i); everything else it names is read
uint32_t zg_seq_op_writes(uint32_t tag) {
    switch (tag) {
        case ZG_OP_NORM: return 1u | (1u << 4) | (1u << 6);   // a chained second destination and a token-shift state, when named
        case ZG_OP_WINDOW_ATTENTION: return 1u | (1u << 2);
        case ZG_OP_CAUSAL_CONV: return 1u | (1u << 3);
        case ZG_OP_DELTA_RULE: return 1u | (1u << 6);
        case ZG_OP_MOE_FFN: return 1u | (1u << 4);
        default: return tag >= ZG_OP_SSM_SCAN ? zg_rec_op_writes(tag) : (tag >= ZG_OP_TOKEN_SHIFT ? zg_mix_op_writes(tag) : 1u);
    }
}

// f32 slots of the shared activation scratch this op needs (0: none): a LINEAR over bfloat16 weights with more rows than the
// row kernels take runs on the tensor cores (dense_gemm.cu) from a bf16 copy of its input.  ZG_DENSE_GEMM=0 keeps the exact tile.
// window shares per (token, head) of a WINDOW_ATTENTION step: few pairs and a long window (decode) spread over more CTAs
static uint32_t attention_splits(const ZgSeqOp& s) {
    const uint32_t pairs = s.n[0] * s.n[1], window = s.n[5];
    if (s.n[3] % 4 || pairs >= 128 || window < 128 || (s.n[0] >= (uint32_t)kWaTiledMinTokens && s.n[3] <= 128)) return 1;   // the tiled prefill kernel splits nothing
    uint32_t S = (256 + pairs - 1) / pairs;
    if (S > window / 32) S = window / 32;
    return S < 2 ? 1 : (S > 16 ? 16 : S);
}
size_t zg_seq_op_scratch_elems(const ZgOp& op, float* const* bufs) {
    if (op.tag >= ZG_OP_SSM_SCAN) return zg_rec_op_scratch_elems(op);
    if (op.tag >= ZG_OP_TOKEN_SHIFT) return zg_mix_op_scratch_elems(op);
    if (op.tag == ZG_OP_WINDOW_ATTENTION) {
        const uint32_t S = attention_splits(op.u.seq);
        return S > 1 ? (size_t)op.u.seq.n[0] * op.u.seq.n[1] * S * (4 + op.u.seq.n[3]) : 0;
    }
    if (op.tag == ZG_OP_DELTA_RULE) {                  // the prepared per-token rows of the prefill form
        const ZgSeqOp& d = op.u.seq;
        return d.n[0] >= (uint32_t)kDeltaPrepMinTokens && d.n[3] <= (uint32_t)kWalkMaxDim ? (size_t)d.n[0] * d.n[1] * (3 * delta_walk_slices(d.n[3]) * kWalkRows + 4) : 0;
    }
    if (!dense_gemm_enabled() || op.tag != ZG_OP_LINEAR || op.u.seq.n[5] != ZG_W_BF16) return 0;
    const ZgSeqOp& s = op.u.seq;
    if (!zg_dense_gemm_usable(wptr<bf16>(bufs, s.buf[2], s.off[0]), s.n[0], s.n[1], s.n[2])) return 0;
    return zg_dense_gemm_scratch_elems(s.n[0], s.n[2]);
}

bool zg_launch_seq_op(ZgCudaCtx* ctx, const ZgOp& op, float* const* bufs, float* scratch, cudaStream_t st) {
    (void)ctx;
    const ZgSeqOp& s = op.u.seq;
    switch (op.tag) {
        case ZG_OP_EMBED:
            ZG_SEQ_WDT(s.n[2], launch_pdl(k_embed<WT>, dim3(s.n[0]), dim3(128), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], wptr<WT>(bufs, s.buf[2], s.off[0]), s.n[1], s.f[0],
                                          s.n[3] ? wptr<WT>(bufs, s.buf[2], s.off[1]) : nullptr));
            ZG_SEQ_CHECK();
            return true;
        case ZG_OP_LINEAR: {
            const uint32_t M = s.n[0], N = s.n[1], K = s.n[2];
            float* dst = bufs[s.buf[0]] + s.off[3];
            const float* src = bufs[s.buf[1]] + s.off[2];
            const bool has_bias = s.buf[3] != ZG_NO_BUF;
            const float* slot_ctl = s.n[7] ? (const float*)bufs[s.buf[4]] : (const float*)nullptr;      // the source is the slot's part of a state buffer
            if (scratch && zg_seq_op_scratch_elems(op, bufs))
                return zg_dense_gemm_launch(wptr<bf16>(bufs, s.buf[2], s.off[0]), has_bias ? wptr<bf16>(bufs, s.buf[3], s.off[1]) : nullptr, src, dst, M, N, K,
                                            s.n[3], s.n[4], scratch, st, s.n[6], s.f[0], slot_ctl, s.n[7]);
            ZG_SEQ_WDT(s.n[5], {
                const WT* W = wptr<WT>(bufs, s.buf[2], s.off[0]);
                const WT* b = has_bias ? wptr<WT>(bufs, s.buf[3], s.off[1]) : nullptr;
                constexpr uint32_t V = WVec<WT>::n;
                if (M <= kGemvRows) {
                    const size_t xs_bytes = (size_t)M * K * sizeof(float);
                    const bool vec = K % V == 0 && (reinterpret_cast<size_t>(W) & 15) == 0 && xs_bytes <= 48 * 1024;
                    const dim3 grid((N + 7) / 8);
                    if (vec && M == 1) launch_pdl(k_linear_rows_vec<WT, 1>, dim3(grid), dim3(256), xs_bytes, st, dst, src, W, b, M, N, K, s.n[3], s.n[4], s.n[6], s.f[0], slot_ctl, s.n[7]);
                    else if (vec && M <= 4) launch_pdl(k_linear_rows_vec<WT, 4>, dim3(grid), dim3(256), xs_bytes, st, dst, src, W, b, M, N, K, s.n[3], s.n[4], s.n[6], s.f[0], slot_ctl, s.n[7]);
                    else if (vec) launch_pdl(k_linear_rows_vec<WT, 8>, dim3(grid), dim3(256), xs_bytes, st, dst, src, W, b, M, N, K, s.n[3], s.n[4], s.n[6], s.f[0], slot_ctl, s.n[7]);
                    else launch_pdl(k_linear_rows<WT>, dim3(grid), dim3(256), 0, st, dst, src, W, b, M, N, K, s.n[3], s.n[4], s.n[6], s.f[0], slot_ctl, s.n[7]);
                } else {
                    const dim3 grid((N + kTN - 1) / kTN, (M + kTM - 1) / kTM);
                    k_linear_tile<WT><<<grid, 256, 0, st>>>(dst, src, W, b, M, N, K, s.n[3], s.n[4], s.n[6], s.f[0], slot_ctl, s.n[7]);
                }
            });
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_NORM: {
            const float* res = s.buf[3] != ZG_NO_BUF ? bufs[s.buf[3]] : nullptr;
            float* dst2 = s.buf[4] != ZG_NO_BUF ? bufs[s.buf[4]] : nullptr;
            float* shift_state = s.buf[6] != ZG_NO_BUF ? bufs[s.buf[6]] : nullptr;
            const uint32_t avg_terms = s.n[5];             // averaged source: buf 4 receives the average instead of a chained norm
            if (((s.n[2] | (dst2 ? s.n[4] : 0u)) & 24u) || s.n[7]) {   // Dynamic Tanh or the plain residual step somewhere in the launch, or two sources
#define ZG_NORM_ANY(KEEP_, THREADS_)                                                                                                               \
    ZG_SEQ_WDT(s.n[3], launch_pdl(k_norm_any<WT, KEEP_, THREADS_>, dim3(s.n[0]), dim3(THREADS_), 0, st, bufs[s.buf[0]] + s.off[3], (const float*)bufs[s.buf[1]], \
                                  (s.n[2] & 16u) ? (const WT*)nullptr : wptr<WT>(bufs, s.buf[2], s.off[0]), res, s.n[1], s.n[2], s.f[0], dst2,                \
                                  dst2 && !(s.n[4] & 16u) ? wptr<WT>(bufs, s.buf[5], s.off[1]) : (const WT*)nullptr, s.n[4], s.f[1],                         \
                                  s.n[7] ? (const float*)bufs[s.buf[6]] : (const float*)nullptr, s.n[7] ? wptr<WT>(bufs, s.buf[2], s.off[2]) : (const WT*)nullptr))
                if (s.n[0] >= 64 || s.n[1] > 4096)
                    ZG_SEQ_WDT(s.n[3], launch_pdl(k_norm_any_rows<WT>, dim3(s.n[0]), dim3(256), 0, st, bufs[s.buf[0]] + s.off[3], (const float*)bufs[s.buf[1]],
                                                  (s.n[2] & 16u) ? (const WT*)nullptr : wptr<WT>(bufs, s.buf[2], s.off[0]), res, s.n[1], s.n[2], s.f[0], dst2,
                                                  dst2 && !(s.n[4] & 16u) ? wptr<WT>(bufs, s.buf[5], s.off[1]) : (const WT*)nullptr, s.n[4], s.f[1],
                                                  s.n[7] ? (const float*)bufs[s.buf[6]] : (const float*)nullptr, s.n[7] ? wptr<WT>(bufs, s.buf[2], s.off[2]) : (const WT*)nullptr));
                else if (s.n[1] <= 1024) ZG_NORM_ANY(4, 256);
                else if (s.n[1] <= 2048) ZG_NORM_ANY(8, 256);
                else ZG_NORM_ANY(8, 512);                      // up to 4096 columns in registers; wider rows are walked from memory
#undef ZG_NORM_ANY
                ZG_SEQ_CHECK();
                return true;
            }
            if (avg_terms) dst2 = nullptr;
            ZG_SEQ_WDT(s.n[3], launch_pdl(k_norm<WT>, dim3(s.n[0]), dim3(256), 0, st, bufs[s.buf[0]] + s.off[3], bufs[s.buf[1]], wptr<WT>(bufs, s.buf[2], s.off[0]), res, s.n[1], s.n[2], s.f[0],
                                          dst2, dst2 ? wptr<WT>(bufs, s.buf[5], s.off[1]) : nullptr, s.n[4], s.f[1],
                                          shift_state ? wptr<WT>(bufs, s.buf[dst2 ? 5 : 2], s.off[2]) : nullptr, shift_state, shift_state ? bufs[s.buf[7]] : nullptr,
                                          avg_terms ? wptr<WT>(bufs, s.buf[2], s.off[4]) : nullptr, avg_terms, s.n[6], avg_terms ? bufs[s.buf[4]] : nullptr));
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_WINDOW_ATTENTION: {
            const uint32_t T = s.n[0], H = s.n[1], G = s.n[2], dim = s.n[3];
            launch_pdl(k_ring_append, dim3(T), dim3(128), 0, st, bufs[s.buf[2]], bufs[s.buf[1]], bufs[s.buf[4]], s.off[1], s.n[4], G * dim, s.n[6]);
            ZG_SEQ_CHECK();
            const size_t width = (size_t)G * dim;
            const bool vec = dim % 4 == 0 && s.off[0] % 4 == 0 && s.n[4] % 4 == 0 && width % 4 == 0 && (reinterpret_cast<uintptr_t>(bufs[s.buf[1]]) & 15) == 0 &&
                             (reinterpret_cast<uintptr_t>(bufs[s.buf[2]]) & 15) == 0;
            if (vec && s.off[2] % 4 == 0 && T >= kWaTiledMinTokens && dim <= 128) {
                switch ((dim + 15) / 16) {
                    case 1: launch_window_attention_tiled<1>(s, bufs, st); break;
                    case 2: launch_window_attention_tiled<2>(s, bufs, st); break;
                    case 3: launch_window_attention_tiled<3>(s, bufs, st); break;
                    case 4: launch_window_attention_tiled<4>(s, bufs, st); break;
                    case 5: launch_window_attention_tiled<5>(s, bufs, st); break;
                    case 6: launch_window_attention_tiled<6>(s, bufs, st); break;
                    case 7: launch_window_attention_tiled<7>(s, bufs, st); break;
                    default: launch_window_attention_tiled<8>(s, bufs, st); break;
                }
            } else if (vec) {
                const uint32_t CH = dim > 128 ? 2 : 1;
                uint32_t LK = 1;
                while (LK * 4 * CH < dim) LK <<= 1;
                const uint32_t S = scratch ? attention_splits(s) : 1;
                float* part = S > 1 ? scratch : nullptr;
                const uint32_t nw = S > 1 ? 4 : (T * H <= 64 ? 16 : (T * H <= 1024 ? 8 : 4));
                const size_t smem = (size_t)nw * (4 + dim) * sizeof(float);
                if (CH == 1)
                    launch_pdl(k_window_attention_v<1>, dim3(T * H, S), dim3(nw * 32), smem, st, bufs[s.buf[0]], bufs[s.buf[1]], bufs[s.buf[2]], bufs[s.buf[3]], bufs[s.buf[4]], H, G, dim, LK,
                                                                        s.n[4], s.off[0], s.off[2], s.n[5], s.n[6], s.f[0], s.f[1], part);
                else
                    launch_pdl(k_window_attention_v<2>, dim3(T * H, S), dim3(nw * 32), smem, st, bufs[s.buf[0]], bufs[s.buf[1]], bufs[s.buf[2]], bufs[s.buf[3]], bufs[s.buf[4]], H, G, dim, LK,
                                                                        s.n[4], s.off[0], s.off[2], s.n[5], s.n[6], s.f[0], s.f[1], part);
                if (S > 1) {
                    ZG_SEQ_CHECK();
                    launch_pdl(k_window_attention_merge, dim3(T * H), dim3(128), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], part, H, dim, S, s.n[4], s.off[2]);
                }
            } else {
                const uint32_t warps = 4;
                launch_pdl(k_window_attention, dim3((T * H + warps - 1) / warps), dim3(warps * 32), warps * dim * sizeof(float), st, 
                    bufs[s.buf[0]], bufs[s.buf[1]], bufs[s.buf[2]], bufs[s.buf[3]], bufs[s.buf[4]], T, H, G, dim, s.n[4], s.off[0], s.off[2], s.n[5], s.n[6], s.f[0], s.f[1]);
            }
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_CAUSAL_CONV: {
            const uint32_t T = s.n[0], C = s.n[1], taps = s.n[2];
            float* dst = bufs[s.buf[0]] + s.off[2];
            const float* src = bufs[s.buf[1]] + s.off[1];
            const size_t n = (size_t)T * C;
            ZG_SEQ_WDT(s.n[6], launch_pdl(k_causal_conv<WT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, dst, src, wptr<WT>(bufs, s.buf[2], s.off[0]), bufs[s.buf[3]], bufs[s.buf[4]],
                                                                                          T, C, taps, s.n[3], s.n[4], s.n[5], (uint32_t)(T == 1 && taps > 1),
                                                                                          s.n[7] ? wptr<WT>(bufs, s.buf[2], s.off[3]) : nullptr));
            ZG_SEQ_CHECK();
            if (taps > 1 && T > 1) {
                launch_pdl(k_conv_advance, dim3((C + 127) / 128), dim3(128), 0, st, bufs[s.buf[3]], src, bufs[s.buf[4]], T, C, taps, s.n[3]);
                ZG_SEQ_CHECK();
            }
            return true;
        }
        case ZG_OP_DELTA_RULE: {
            const uint32_t T = s.n[0], H = s.n[1], G = s.n[2], dim = s.n[3], vdim = s.n[4];
            const uint32_t form = s.n[10], dst_rs = s.n[11] ? s.n[11] : H * vdim;
            const float inv_tau = (form & kDeltaSigmoidDecay) ? 1.0f / s.f[3] : 0.0f, out_scale = (form & kDeltaOutScale) ? s.f[4] : 1.0f;
            float* dst = bufs[s.buf[0]] + s.n[12];
            const float* betab = (form & kDeltaPlain) ? nullptr : bufs[s.buf[2]];
            const uint32_t RS = zg_delta_row_slices(dim), cols = kDeltaThreads / RS;
            const size_t smem = ((size_t)3 * kDeltaTile * RS * kDeltaRows + kDeltaTile) * sizeof(float);
            const dim3 grid((vdim + cols - 1) / cols, H);
            if (scratch && T >= (uint32_t)kDeltaPrepMinTokens && dim <= (uint32_t)kWalkMaxDim) {
                const uint32_t WS = delta_walk_slices(dim), dpad = WS * kWalkRows, wcols = kWalkThreads / WS;
                const size_t walk_smem = (size_t)2 * kDeltaTile * (3 * dpad + 4) * sizeof(float);
                ZG_SEQ_WDT(s.n[9], launch_pdl(k_delta_prepare<WT>, dim3((T * H + 3) / 4), dim3(128), 0, st, scratch, bufs[s.buf[1]], betab, bufs[s.buf[3]],
                                              wptr<WT>(bufs, s.buf[5], 0), T, H, G, dim, dpad, s.off[0], s.off[1], s.off[3], s.off[4], s.off[5], s.n[5], s.n[6], s.n[7], s.f[1], s.f[2],
                                              form, inv_tau));
                ZG_SEQ_CHECK();
#define ZG_WALK(RS_)                                                                                                                            \
    case RS_:                                                                                                                                   \
        if (form & kDeltaPlain) {                                                                                                               \
            if (walk_smem > 48 * 1024) cudaFuncSetAttribute(k_delta_walk<RS_, true>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)walk_smem); \
            launch_pdl(k_delta_walk<RS_, true>, dim3((vdim + wcols - 1) / wcols, H), dim3(kWalkThreads), walk_smem, st, dst, bufs[s.buf[1]],    \
                       scratch, bufs[s.buf[6]], bufs[s.buf[7]], T, H, dim, vdim, s.off[2], s.n[5], dst_rs);                                     \
        } else {                                                                                                                                \
            if (walk_smem > 48 * 1024) cudaFuncSetAttribute(k_delta_walk<RS_, false>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)walk_smem); \
            launch_pdl(k_delta_walk<RS_, false>, dim3((vdim + wcols - 1) / wcols, H), dim3(kWalkThreads), walk_smem, st, dst, bufs[s.buf[1]],   \
                       scratch, bufs[s.buf[6]], bufs[s.buf[7]], T, H, dim, vdim, s.off[2], s.n[5], dst_rs);                                     \
        }                                                                                                                                       \
        break;
                switch (WS) { ZG_WALK(1) ZG_WALK(2) ZG_WALK(4) ZG_WALK(8) ZG_WALK(16) default: ZG_WALK(32) }
#undef ZG_WALK
            } else ZG_SEQ_WDT(s.n[9], {
                if (smem > 48 * 1024) cudaFuncSetAttribute(k_delta_rule<WT>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);
                launch_pdl(k_delta_rule<WT>, dim3(grid), dim3(kDeltaThreads), smem, st, dst, bufs[s.buf[1]], betab, bufs[s.buf[3]], wptr<WT>(bufs, s.buf[5], 0), bufs[s.buf[6]],
                                                                  bufs[s.buf[7]], T, H, G, dim, vdim, RS, s.off[0], s.off[1], s.off[2], s.off[3], s.off[4], s.off[5],
                                                                  s.n[5], s.n[6], s.n[7], s.f[1], s.f[2], form, inv_tau, dst_rs);
            });
            ZG_SEQ_CHECK();
            ZG_SEQ_WDT(s.n[9], launch_pdl(k_delta_out<WT>, dim3((T * H + 3) / 4), dim3(128), 0, st, dst, bufs[s.buf[4]] + s.off[7], wptr<WT>(bufs, s.buf[5], 0), T * H, H, vdim, s.n[8], s.off[6], s.f[0],
                                                           dst_rs, (uint32_t)((form & kDeltaSiluGate) != 0), out_scale));
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_ROUTE: {
            const uint32_t T = s.n[0], NE = s.n[1];
            const uint32_t groups = s.n[5] == 2 && s.n[6] > 1 ? s.n[6] : 0;
            ZG_SEQ_WDT(s.n[4], launch_pdl(k_route<WT>, dim3((T + 3) / 4), dim3(128), 4 * (NE + groups) * sizeof(float), st, bufs[s.buf[0]], bufs[s.buf[1]] + s.off[1], wptr<WT>(bufs, s.buf[2], s.off[0]), T, NE,
                                                                                         s.n[2], s.n[3], s.n[5], groups, s.n[7]));
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_MOE_FFN: {
            const uint32_t T = s.n[0], D = s.n[1], ff = s.n[2], E = s.n[3], top = s.n[4];
            if (moe_grouped(s, bufs)) {
                const MoeLayout L = moe_layout(T, D, ff, E, top);
                float* sc = bufs[s.buf[4]];
                int* tile_group = reinterpret_cast<int*>(sc + L.tile_group);
                int* row_pair = reinterpret_cast<int*>(sc + L.row_pair);
                int* pos_of_pair = reinterpret_cast<int*>(sc + L.pos_of_pair);
                k_moe_sort<<<1, 1024, 0, st>>>(bufs[s.buf[2]], tile_group, row_pair, pos_of_pair, T * top, E, L.R);
                ZG_SEQ_CHECK();
                k_moe_gather<<<L.R, 256, 0, st>>>(reinterpret_cast<uint32_t*>(sc + L.xs), bufs[s.buf[1]], row_pair, D, L.Dp / 2, top);
                ZG_SEQ_CHECK();
                if (!zg_dense_gemm_grouped_launch(wptr<bf16>(bufs, s.buf[3], s.off[0]), E, sc + L.xs, L.R, L.Dp, tile_group, sc + L.g, ff, D, ff, st) ||
                    !zg_dense_gemm_grouped_launch(wptr<bf16>(bufs, s.buf[3], s.off[1]), E, sc + L.xs, L.R, L.Dp, tile_group, sc + L.u, ff, D, ff, st)) return false;
                k_moe_act<<<L.R, 256, 0, st>>>(reinterpret_cast<uint32_t*>(sc + L.yb), sc + L.g, sc + L.u, row_pair, ff, L.Fp / 2, s.f[0], s.f[1], s.f[2]);
                ZG_SEQ_CHECK();
                if (!zg_dense_gemm_grouped_launch(wptr<bf16>(bufs, s.buf[3], s.off[2]), E, sc + L.yb, L.R, L.Fp, tile_group, sc + L.z, D, ff, D, st)) return false;
                k_moe_combine<<<T, 256, 0, st>>>(bufs[s.buf[0]], bufs[s.buf[1]], sc + L.z, bufs[s.buf[2]], pos_of_pair, D, top);
                ZG_SEQ_CHECK();
                return true;
            }
            ZG_SEQ_WDT(s.n[5], {
                if (E && ff) {
                    const uint32_t stage = (size_t)D * 4 <= 48 * 1024 ? 1u : 0u;
                    launch_pdl(k_moe_up<WT>, dim3(dim3((ff + 7) / 8, T * top)), dim3(256), stage ? D * sizeof(float) : 0, st, bufs[s.buf[4]], bufs[s.buf[1]], bufs[s.buf[2]], wptr<WT>(bufs, s.buf[3], s.off[0]),
                                                                           wptr<WT>(bufs, s.buf[3], s.off[1]), D, ff, E, top, s.f[0], s.f[1], s.f[2], stage);
                    ZG_COUNT_LAUNCH();
                }
                launch_pdl(k_moe_down<WT>, dim3(dim3((D + 7) / 8, T)), dim3(256), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], bufs[s.buf[4]], bufs[s.buf[2]], wptr<WT>(bufs, s.buf[3], s.off[2]), D, ff, E, top);
            });
            ZG_SEQ_CHECK();
            return true;
        }
        default:
            return op.tag >= ZG_OP_SSM_SCAN ? zg_launch_rec_op(op, bufs, scratch, st) : zg_launch_mix_op(op, bufs, scratch, st);
    }
}
