// Sequence-model DeviceOps ZG_OP_TOKEN_SHIFT .. ZG_OP_POLY_NORM (parameter packs in include/zgml_cuda.h): the pieces of
// decoder stacks whose mixers attend over a per-sequence CACHE of keys and values (or of one latent that serves as both) —
// token shift, a learned average over the depth of the stack, rotary positions, the cache append, softmax attention over
// the cache with grouped heads / several score maps per head / causal, sliding and block masks, the differential
// combination of two maps, sigmoid gates, block-diagonal (per-head) products and the PolyNorm activation.
// Everything here is f32: positions and angles, scores and softmax weights, norms, gates and the sums.
#include "seq_common.cuh"

#include <math.h>

namespace {

// ── TOKEN_SHIFT ──────────────────────────────────────────────────────────────────────────────────────────────────
// Thread (0, c) alone touches state[c]: it reads the previous step's last row there and then replaces it.
template <typename WT>
__global__ void k_token_shift(float* __restrict__ dst, const float* __restrict__ src, const WT* __restrict__ mix, float* __restrict__ state,
                              const float* __restrict__ ctl, uint32_t T, uint32_t D) {
    pdl_enter();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (size_t)T * D) return;
    const uint32_t t = (uint32_t)(e / D), c = (uint32_t)(e % D);
    float* st = state + (size_t)ctl_word(ctl, ZG_CTL_SLOT) * D;
    const float h = src[e];
    const float prev = t ? src[e - D] : st[c];
    dst[e] = fmaf(prev - h, wld(mix, c), h);
    if (t == 0) st[c] = src[(size_t)(T - 1) * D + c];
}

// ── DEPTH_MIX ────────────────────────────────────────────────────────────────────────────────────────────────────
template <typename WT>
__global__ void k_depth_mix(float* __restrict__ dst, const float* __restrict__ hist, const WT* __restrict__ coeff, uint32_t n, uint32_t terms,
                            uint32_t stride) {
    pdl_enter();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= n) return;
    float acc = 0.0f;
    for (uint32_t j = 0; j < terms; j++) acc = fmaf(wld(coeff, j), hist[(size_t)j * stride + e], acc);
    dst[e] = acc;
}

// ── ROTARY ───────────────────────────────────────────────────────────────────────────────────────────────────────
// The frequency is the f32 rounding of base^(-2i / dims); the angle p * f and its sine and cosine are f32.
__device__ __forceinline__ void rotary_angle(uint32_t pos, uint32_t i, uint32_t dims, float base, float& sn, float& cs) {
    const float freq = (float)pow((double)base, -2.0 * (double)i / (double)dims);
    sincosf((float)pos * freq, &sn, &cs);
}
// With `freqs` (dims / 2 values) the pair's frequency comes from that table: a schedule the caller evaluated.
__global__ void k_rotary(float* x, const float* src, const float* __restrict__ ctl, uint32_t T, uint32_t heads, uint32_t head_stride,
                         uint32_t row_stride, uint32_t dims, uint32_t layout, uint32_t src_hs, uint32_t src_rs, float base, const float* __restrict__ freqs) {
    pdl_enter();
    const uint32_t half = dims / 2;
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (size_t)T * heads * half) return;
    const uint32_t i = (uint32_t)(e % half), hd = (uint32_t)((e / half) % heads), t = (uint32_t)(e / ((size_t)half * heads));
    float sn, cs;
    if (freqs) sincosf((float)((uint32_t)ctl_word(ctl, ZG_CTL_POS) + t) * freqs[i], &sn, &cs);
    else rotary_angle((uint32_t)ctl_word(ctl, ZG_CTL_POS) + t, i, dims, base, sn, cs);
    float* v = x + (size_t)t * row_stride + (size_t)hd * head_stride;
    const float* sv = src + (size_t)t * src_rs + (size_t)hd * src_hs;
    const uint32_t a = layout == 0 ? 2 * i : i, b = layout == 0 ? 2 * i + 1 : i + half;
    const float u = sv[a], w = sv[b];
    v[a] = u * cs - w * sn;
    v[b] = w * cs + u * sn;
}

// ── CACHE_APPEND: one CTA per token ──────────────────────────────────────────────────────────────────────────────
// A cache row is [normed | rotated | plain]: the first `normed` columns are divided by their root mean square and weighted
// (a latent), the next `rot` columns get the token's rotary position (a key part shared by the heads), the rest is copied.
template <typename WT>
__global__ void k_cache_append(float* __restrict__ cache, const float* __restrict__ src, const float* __restrict__ ctl, const WT* __restrict__ nw_,
                               uint32_t cols, uint32_t src_rs, uint32_t width, uint32_t R, uint32_t normed, uint32_t rot, uint32_t layout, float eps,
                               float base, uint32_t norm_group, float* qsrc, const WT* __restrict__ qw, uint32_t q_heads, uint32_t temp_every, float temp_coef,
                               uint32_t hrot, const float* __restrict__ freqs) {
    pdl_enter();
    __shared__ float sh[32];
    extern __shared__ float cs_sn[];                   // head rotary: cosine | sine of the token's hrot / 2 angles, shared by all heads
    const uint32_t t = blockIdx.x;
    const uint32_t pos = (uint32_t)ctl_word(ctl, ZG_CTL_POS) + t, slot = (uint32_t)ctl_word(ctl, ZG_CTL_SLOT);
    float* row = cache + ((size_t)slot * R + pos % R) * width;
    const float* s = src + (size_t)t * src_rs;
    if (hrot) {
        // Every key head (and query head) is first turned by the token's position on its first hrot values, then divided by the
        // root mean square of the TURNED vector and weighted: rotary and norm of a head in one pass over it.  One warp per head;
        // a lane turns whole pairs, so turning in place (the query heads) has no hazard between lanes.
        const uint32_t hh = hrot / 2;
        for (uint32_t i = threadIdx.x; i < hh; i += blockDim.x) {
            float sn, cs;
            if (freqs) sincosf((float)pos * freqs[i], &sn, &cs); else rotary_angle(pos, i, hrot, base, sn, cs);
            cs_sn[i] = cs; cs_sn[hh + i] = sn;
        }
        __syncthreads();
        const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
        const uint32_t n_key = normed / norm_group;
        const float temp = temp_every ? fmaf(temp_coef, logf((float)((pos + 1) / temp_every) + 1.0f), 1.0f) : 1.0f;
        for (uint32_t hd = warp; hd < n_key + q_heads; hd += nw) {
            const bool key = hd < n_key;
            const float* v = key ? s + (size_t)hd * norm_group : qsrc + (size_t)t * src_rs + (size_t)(hd - n_key) * norm_group;
            float* d = key ? row + (size_t)hd * norm_group : qsrc + (size_t)t * src_rs + (size_t)(hd - n_key) * norm_group;
            const WT* w = key ? nw_ : qw;
            float q = 0.0f;
            for (uint32_t i = lane; i < hh; i += 32) {
                const uint32_t a = layout == 0 ? 2 * i : i, b = layout == 0 ? 2 * i + 1 : i + hh;
                const float u = v[a], x = v[b], ru = u * cs_sn[i] - x * cs_sn[hh + i], rx = x * cs_sn[i] + u * cs_sn[hh + i];
                d[a] = ru; d[b] = rx;
                q = fmaf(ru, ru, fmaf(rx, rx, q));
            }
            for (uint32_t c = hrot + lane; c < norm_group; c += 32) { const float x = v[c]; d[c] = x; q = fmaf(x, x, q); }
            const float mult = (key ? 1.0f : temp) / sqrtf(warp_sum(q) / (float)norm_group + eps);
            __syncwarp();
            for (uint32_t c = lane; c < norm_group; c += 32) d[c] = d[c] * mult * wld(w, c);
        }
        for (uint32_t c = normed + rot + threadIdx.x; c < cols; c += blockDim.x) row[c] = s[c];
        return;
    }
    if (normed && norm_group) {                        // key heads: every group of norm_group columns by its own root mean square, one warp each
        const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
        for (uint32_t g0 = warp * norm_group; g0 < normed; g0 += nw * norm_group) {
            float q = 0.0f;
            for (uint32_t c = lane; c < norm_group; c += 32) q = fmaf(s[g0 + c], s[g0 + c], q);
            const float inv = 1.0f / sqrtf(warp_sum(q) / (float)norm_group + eps);
            for (uint32_t c = lane; c < norm_group; c += 32) row[g0 + c] = s[g0 + c] * inv * wld(nw_, c);
        }
    } else if (normed) {
        float q = 0.0f;
        for (uint32_t c = threadIdx.x; c < normed; c += blockDim.x) q = fmaf(s[c], s[c], q);
        const float inv = 1.0f / sqrtf(block_sum(q, sh) / (float)normed + eps);
        for (uint32_t c = threadIdx.x; c < normed; c += blockDim.x) row[c] = s[c] * inv * wld(nw_, c);
    }
    const uint32_t half = rot / 2;
    for (uint32_t i = threadIdx.x; i < half; i += blockDim.x) {
        float sn, cs;
        rotary_angle(pos, i, rot, base, sn, cs);
        const uint32_t a = normed + (layout == 0 ? 2 * i : i), b = normed + (layout == 0 ? 2 * i + 1 : i + half);
        const float u = s[a], w = s[b];
        row[a] = u * cs - w * sn;
        row[b] = w * cs + u * sn;
    }
    for (uint32_t c = normed + rot + threadIdx.x; c < cols; c += blockDim.x) row[c] = s[c];
    if (q_heads) {     // the step's QUERY heads are normed in place by the same launch (per head, one shared weight), times a temperature that grows with the position
        const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
        const float temp = temp_every ? fmaf(temp_coef, logf((float)((pos + 1) / temp_every) + 1.0f), 1.0f) : 1.0f;
        float* qrow = qsrc + (size_t)t * src_rs;
        for (uint32_t hd = warp; hd < q_heads; hd += nw) {
            float* v = qrow + (size_t)hd * norm_group;
            float q = 0.0f;
            for (uint32_t c = lane; c < norm_group; c += 32) q = fmaf(v[c], v[c], q);
            const float mult = temp / sqrtf(warp_sum(q) / (float)norm_group + eps);
            for (uint32_t c = lane; c < norm_group; c += 32) v[c] = v[c] * wld(qw, c) * mult;
        }
    }
}

// ── CACHED_ATTENTION ─────────────────────────────────────────────────────────────────────────────────────────────
// first position a query at p can see
__device__ __forceinline__ uint32_t mask_low(uint32_t p, uint32_t kind, uint32_t size) {
    if (kind == 1) return p + 1 >= size ? p + 1 - size : 0;
    if (kind == 2) return p - p % size;
    return 0;
}
struct CaArgs {
    float* dst; const float* q; const float* kc; const float* vc; const float* ctl;
    uint32_t T, H, G, maps, dk, dv, q_rs, q_off, kw, k_off, vw, v_off, R, kind, size;
    float scale;
    const float* tab;      // score table [H * maps, tab_rs] by distance, or null
    uint32_t tab_rs, wkind;   // weights: 0 softmax over the visible keys, 1 sigmoid of every visible key (not normalised)
    float cap;             // > 0: the scaled score passes cap * tanh(s / cap)
    const void* sink;      // a learned score per (head, map) that joins the softmax's denominator only, or null
    uint32_t sink_bf16;    // its weight type
    float out_scale;       // the result is multiplied by it
    uint32_t dst_rs;       // row stride of dst (its first column is folded into the pointer)
    uint32_t unslotted;    // the caches belong to the step (rows recomputed by the program), not to a state slot
};
__device__ __forceinline__ uint32_t ca_slot(const CaArgs& a) { return a.unslotted ? 0u : (uint32_t)ctl_word(a.ctl, ZG_CTL_SLOT); }
__device__ __forceinline__ float ca_score(const CaArgs& a, float dot) {
    const float s = dot * a.scale;
    return a.cap > 0.0f ? a.cap * tanhf(s / a.cap) : s;
}
__device__ __forceinline__ float ca_sink(const CaArgs& a, uint32_t hm) {
    return a.sink_bf16 ? __bfloat162float(reinterpret_cast<const bf16*>(a.sink)[hm]) : reinterpret_cast<const float*>(a.sink)[hm];
}
// 1 / (sum + exp(sink - max)): the sink's share of the denominator, in the frame of the running maximum
__device__ __forceinline__ float ca_inv_sum(const CaArgs& a, uint32_t hm, float mx, float l) {
    if (a.sink) l += expf(ca_sink(a, hm) - mx);
    return 1.0f / l;
}
// weight of a visible key under the unnormalised kind
__device__ __forceinline__ float ca_sigmoid(float s) { return __frcp_rn(1.0f + expf(-s)); }
constexpr int kCaMaxDv = 1024;   // 32 channels per lane in the per-query kernel
// Any shape: one warp per (token, head, map); 32 keys at a time, lane = key for the scores, lane = channel for the sum.
__global__ void k_cached_attention(CaArgs a) {
    pdl_enter();
    extern __shared__ float sq[];                      // [warps][dk]
    const uint32_t warp = threadIdx.x >> 5, lane = threadIdx.x & 31, nw = blockDim.x >> 5;
    const uint32_t HM = a.H * a.maps;
    const uint32_t item = blockIdx.x * nw + warp;
    if (item >= a.T * HM) return;
    const uint32_t t = item / HM, hm = item % HM, h = hm / a.maps, m = hm % a.maps, g = h / (a.H / a.G);
    const uint32_t pos0 = (uint32_t)ctl_word(a.ctl, ZG_CTL_POS), slot = ca_slot(a);
    const uint32_t p = pos0 + t, lo = mask_low(p, a.kind, a.size);
    float* q = sq + warp * a.dk;
    const float* qrow = a.q + (size_t)t * a.q_rs + a.q_off + (size_t)hm * a.dk;
    for (uint32_t c = lane; c < a.dk; c += 32) q[c] = qrow[c];
    __syncwarp();
    const float* kbase = a.kc + (size_t)slot * a.R * a.kw + a.k_off + (size_t)(g * a.maps + m) * a.dk;
    const float* vbase = a.vc + (size_t)slot * a.R * a.vw + a.v_off + (size_t)g * a.dv;
    float mx = -INFINITY, l = 0.0f;
    float acc[kCaMaxDv / 32];
#pragma unroll
    for (int i = 0; i < kCaMaxDv / 32; i++) acc[i] = 0.0f;
    for (uint32_t j0 = lo; j0 <= p; j0 += 32) {
        const uint32_t j = j0 + lane;
        float s = -INFINITY;
        if (j <= p) {
            const float* k = kbase + (size_t)(j % a.R) * a.kw;
            float d = 0.0f;
            for (uint32_t c = 0; c < a.dk; c++) d = fmaf(q[c], k[c], d);
            s = ca_score(a, d);
            if (a.tab) s += a.tab[(size_t)hm * a.tab_rs + (p - j)];
        }
        float corr = 1.0f, e;
        if (a.wkind) e = j <= p ? ca_sigmoid(s) : 0.0f;
        else {
            const float m_new = fmaxf(mx, warp_max(s));    // finite: key j0 is visible
            corr = expf(mx - m_new);
            e = j <= p ? expf(s - m_new) : 0.0f;
            l = l * corr + warp_sum(e);
            mx = m_new;
        }
        const uint32_t cnt = min(32u, p - j0 + 1);
#pragma unroll
        for (int i = 0; i < kCaMaxDv / 32; i++) acc[i] *= corr;
        for (uint32_t jj = 0; jj < cnt; jj++) {
            const float pj = __shfl_sync(0xffffffffu, e, jj);
            const float* v = vbase + (size_t)((j0 + jj) % a.R) * a.vw;
#pragma unroll
            for (int i = 0; i < kCaMaxDv / 32; i++) {
                const uint32_t c = lane + 32 * i;
                if (c < a.dv) acc[i] = fmaf(pj, v[c], acc[i]);
            }
        }
    }
    const float inv = (a.wkind ? 1.0f : ca_inv_sum(a, hm, mx, l)) * a.out_scale;
    float* out = a.dst + (size_t)t * a.dst_rs + (size_t)hm * a.dv;
#pragma unroll
    for (int i = 0; i < kCaMaxDv / 32; i++) {
        const uint32_t c = lane + 32 * i;
        if (c < a.dv) out[c] = acc[i] * inv;
    }
}


// Tiled form (16-byte aligned shapes): flash tiling in f32.  The query ROWS of a tile are (token, head of the key group)
// pairs, so the heads that share a key head — all heads of a latent attention, the group of a grouped one — meet every key
// tile once, in a prompt (64 rows = 64 / heads-per-group tokens) and in decoding alike (a few tokens x the group's heads).
// One CTA owns 64 rows of one (key head, map) and one slice of up to 16 OC value columns, and walks the key tiles its rows'
// masks reach: the scores accumulate over 64-wide slices of the key dimension (any dk), thread (ty, tx) of 16 x 16 holding
// rows 4 ty .. 4 ty + 3 against keys tx + 16 c; the row statistics of the running softmax are shared through half-warp
// shuffles, the probabilities pass through shared memory, value columns tx + 16 c accumulate in registers.  With `splits`
// > 1 (few rows, long caches: decoding) the keys are dealt in contiguous ranges to gridDim.z CTAs, each leaving (max, sum,
// unnormalised output) per row for k_cached_attention_merge; a range may be shorter than a tile (its other keys are neither
// loaded nor counted), since what bounds such a step is how many SMs pull on the cache, not the arithmetic.
constexpr int kCtBQ = 64, kCtBK = 64, kCtDS = 64, kCtThreads = 256, kCtMaxSplits = 64, kCtMinShare = 32;
// 16 bytes global -> shared without passing through registers; `on` false writes zeros (nothing is read)
__device__ __forceinline__ void copy16(float* dst, const float* src, bool on) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = on ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
template <int OC>
__global__ void __launch_bounds__(kCtThreads) k_cached_attention_tiled(CaArgs a, uint32_t rh, uint32_t n_tiles, uint32_t splits, float* __restrict__ part) {
    pdl_enter();
    constexpr int DV = 16 * OC, KP = kCtDS + 4, PP = kCtBK + 4;
    extern __shared__ __align__(16) float sm[];
    // The 64-wide slices of the queries and keys are double-buffered: while a slice is multiplied, cp.async brings the next
    // one (of this key tile or the first of the next), so the cache's latency hides behind the arithmetic.  Queries no wider
    // than one slice are loaded once and keep a single buffer.
    const bool q_once = a.dk <= (uint32_t)kCtDS;
    float* Qs = sm;                                    // [1 or 2][64][64]
    float* Ks = Qs + (q_once ? 1 : 2) * kCtBQ * kCtDS; // [2][64][64 + 4]
    float* Ps = Ks + 2 * kCtBK * KP;                   // [64][64 + 4]
    float* Vs = Ps + kCtBQ * PP;                       // [64][DV]
    const uint32_t tid = threadIdx.x, tx = tid & 15, ty = tid >> 4;
    const uint32_t n_vs = (a.dv + DV - 1) / DV;
    const uint32_t tile = n_tiles - 1 - blockIdx.x;    // later rows walk more keys: heaviest first
    const uint32_t gm = blockIdx.y / n_vs, vs = blockIdx.y % n_vs, g = gm / a.maps, m = gm % a.maps;
    const uint32_t pos0 = (uint32_t)ctl_word(a.ctl, ZG_CTL_POS), slot = ca_slot(a);
    const uint32_t total = a.T * rh, r0 = tile * kCtBQ, nq = min((uint32_t)kCtBQ, total - r0);
    const uint32_t p_min = pos0 + r0 / rh, p_max = pos0 + (r0 + nq - 1) / rh;
    const uint32_t k_lo = mask_low(p_min, a.kind, a.size);
    const uint32_t n_keys = p_max - k_lo + 1, per = (n_keys + splits - 1) / splits;
    const uint32_t k_begin = k_lo + blockIdx.z * per, k_end = min(p_max + 1, k_begin + per);   // this CTA's keys [k_begin, k_end)
    const float* kbase = a.kc + (size_t)slot * a.R * a.kw + a.k_off + (size_t)gm * a.dk;
    const float* vbase = a.vc + (size_t)slot * a.R * a.vw + a.v_off + (size_t)g * a.dv + (size_t)vs * DV;
    const uint32_t v_cols = min((uint32_t)DV, a.dv - vs * DV);
    uint32_t p_r[4], lo_r[4];
    bool ok_r[4];
    const float* tab_r[4];                             // the row's line of the score table, so that tab_r[p - j] is the entry of key j
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t r = r0 + 4 * ty + i;
        ok_r[i] = r < total;
        p_r[i] = pos0 + (ok_r[i] ? r / rh : 0);
        lo_r[i] = mask_low(p_r[i], a.kind, a.size);
        tab_r[i] = a.tab ? a.tab + (size_t)((g * rh + (ok_r[i] ? r % rh : 0)) * a.maps + m) * a.tab_rs : nullptr;
    }
    auto load_q = [&](uint32_t d0, uint32_t stage) {
        for (uint32_t i = tid; i < kCtBQ * (kCtDS / 4); i += kCtThreads) {
            const uint32_t rr = i / (kCtDS / 4), c4 = i % (kCtDS / 4), r = r0 + rr;
            const bool on = r < total && d0 + 4 * c4 < a.dk;
            const float* src = on ? a.q + (size_t)(r / rh) * a.q_rs + a.q_off + (size_t)((g * rh + r % rh) * a.maps + m) * a.dk + d0 + 4 * c4 : a.q;
            copy16(Qs + stage * kCtBQ * kCtDS + rr * kCtDS + 4 * c4, src, on);
        }
    };
    auto load_k = [&](uint32_t s0, uint32_t d0, uint32_t stage) {
        for (uint32_t i = tid; i < kCtBK * (kCtDS / 4); i += kCtThreads) {
            const uint32_t rr = i / (kCtDS / 4), c4 = i % (kCtDS / 4);
            const bool on = s0 + rr < k_end && d0 + 4 * c4 < a.dk;
            copy16(Ks + stage * kCtBK * KP + rr * KP + 4 * c4, on ? kbase + (size_t)((s0 + rr) % a.R) * a.kw + d0 + 4 * c4 : kbase, on);
        }
    };
    auto load_v = [&](uint32_t s0) {
        for (uint32_t i = tid; i < kCtBK * (DV / 4); i += kCtThreads) {
            const uint32_t rr = i / (DV / 4), c4 = i % (DV / 4);
            const bool on = s0 + rr < k_end && 4 * c4 < v_cols;
            copy16(Vs + rr * DV + 4 * c4, on ? vbase + (size_t)((s0 + rr) % a.R) * a.vw + 4 * c4 : vbase, on);
        }
    };
    float o[4][OC], m_run[4], l_run[4];
#pragma unroll
    for (int r = 0; r < 4; r++) {
        m_run[r] = -INFINITY; l_run[r] = 0.0f;
#pragma unroll
        for (int c = 0; c < OC; c++) o[r][c] = 0.0f;
    }
    const uint32_t n_slices = (a.dk + kCtDS - 1) / kCtDS;
    uint32_t it = 0;                                   // slices done so far, over all key tiles: slice `it` sits in stage it & 1
    if (k_begin < k_end) {                             // the first slice of the first tile
        load_q(0, 0);
        load_k(k_begin, 0, 0);
    }
    asm volatile("cp.async.commit_group;" ::: "memory");
    for (uint32_t s0 = k_begin; s0 < k_end; s0 += kCtBK) {
        float sc[4][4];
#pragma unroll
        for (int r = 0; r < 4; r++)
#pragma unroll
            for (int c = 0; c < 4; c++) sc[r][c] = 0.0f;
        for (uint32_t sl = 0; sl < n_slices; sl++, it++) {
            const uint32_t d0 = sl * kCtDS, stage = it & 1;
            __syncthreads();                           // the readers of the other stage (the slice before), of Ps and of Vs (the tile before) are done
            if (sl + 1 < n_slices) {                   // bring the next slice while this one is multiplied
                load_q(d0 + kCtDS, stage ^ 1);
                load_k(s0, d0 + kCtDS, stage ^ 1);
            } else if (s0 + kCtBK < k_end) {
                if (!q_once) load_q(0, stage ^ 1);
                load_k(s0 + kCtBK, 0, stage ^ 1);
            }
            if (sl == 0) load_v(s0);                   // needed only after the tile's last slice
            asm volatile("cp.async.commit_group;" ::: "memory");
            asm volatile("cp.async.wait_group 1;" ::: "memory");   // everything but the group just committed has landed: this slice is there
            __syncthreads();
            const float* Qc = Qs + (q_once ? 0 : stage) * kCtBQ * kCtDS;
            const float* Kc = Ks + stage * kCtBK * KP;
            const uint32_t dn = min((uint32_t)kCtDS, a.dk - d0);
#pragma unroll 2
            for (uint32_t d = 0; d < dn; d += 4) {
                float4 qa[4], ka[4];
#pragma unroll
                for (int r = 0; r < 4; r++) qa[r] = *reinterpret_cast<const float4*>(Qc + (4 * ty + r) * kCtDS + d);
#pragma unroll
                for (int c = 0; c < 4; c++) ka[c] = *reinterpret_cast<const float4*>(Kc + (tx + 16 * c) * KP + d);
#pragma unroll
                for (int r = 0; r < 4; r++)
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        sc[r][c] = fmaf(qa[r].x, ka[c].x, sc[r][c]); sc[r][c] = fmaf(qa[r].y, ka[c].y, sc[r][c]);
                        sc[r][c] = fmaf(qa[r].z, ka[c].z, sc[r][c]); sc[r][c] = fmaf(qa[r].w, ka[c].w, sc[r][c]);
                    }
            }
        }
        if (n_slices == 1) {                           // the values came with this very slice's group: wait for them too
            asm volatile("cp.async.wait_group 0;" ::: "memory");
        }
#pragma unroll
        for (int r = 0; r < 4; r++) {
            const uint32_t row = 4 * ty + r;
            float rmax = -INFINITY;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const uint32_t j = s0 + tx + 16 * c;
                const bool seen = ok_r[r] && j <= p_r[r] && j >= lo_r[r] && j < k_end;
                float sv = seen ? ca_score(a, sc[r][c]) : -INFINITY;
                if (seen && tab_r[r]) sv += tab_r[r][p_r[r] - j];
                sc[r][c] = sv;
                rmax = fmaxf(rmax, sv);
            }
            if (a.wkind) {                             // every visible key weighs sigmoid(score): no running maximum, no sum
#pragma unroll
                for (int c = 0; c < 4; c++) Ps[row * PP + tx + 16 * c] = sc[r][c] == -INFINITY ? 0.0f : ca_sigmoid(sc[r][c]);
                continue;
            }
#pragma unroll
            for (int off = 8; off > 0; off >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, off));
            const float new_m = fmaxf(m_run[r], rmax);
            const float alpha = m_run[r] == -INFINITY ? (new_m == -INFINITY ? 1.0f : 0.0f) : expf(m_run[r] - new_m);
            float rsum = 0.0f;
#pragma unroll
            for (int c = 0; c < 4; c++) {
                const float pv = sc[r][c] == -INFINITY ? 0.0f : expf(sc[r][c] - new_m);
                Ps[row * PP + tx + 16 * c] = pv;
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
        for (int j = 0; j < kCtBK; j++) {
            float pj[4], vj[OC];
#pragma unroll
            for (int r = 0; r < 4; r++) pj[r] = Ps[(4 * ty + r) * PP + j];
#pragma unroll
            for (int c = 0; c < OC; c++) vj[c] = Vs[j * DV + tx + 16 * c];
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < OC; c++) o[r][c] = fmaf(pj[r], vj[c], o[r][c]);
        }
    }
#pragma unroll
    for (int r = 0; r < 4; r++) {
        const uint32_t row = r0 + 4 * ty + r;
        if (!ok_r[r]) continue;
        const uint32_t hm = (g * rh + row % rh) * a.maps + m;
        if (splits == 1) {
            const float inv = (a.wkind ? 1.0f : ca_inv_sum(a, hm, m_run[r], l_run[r])) * a.out_scale;         // every query sees itself
            float* out = a.dst + (size_t)(row / rh) * a.dst_rs + (size_t)hm * a.dv + (size_t)vs * DV;
#pragma unroll
            for (int c = 0; c < OC; c++) if (tx + 16 * c < v_cols) out[tx + 16 * c] = o[r][c] * inv;
        } else {
            float* mine = part + (((size_t)(row / rh) * a.H * a.maps + hm) * splits + blockIdx.z) * (4 + a.dv);
            if (tx == 0 && vs == 0) { mine[0] = m_run[r]; mine[1] = l_run[r]; }
#pragma unroll
            for (int c = 0; c < OC; c++) if (tx + 16 * c < v_cols) mine[4 + (size_t)vs * DV + tx + 16 * c] = o[r][c];
        }
    }
}
// merge of the key shares: CTA (x, y) = 128 value columns y of (token, head, map) x; a share that saw no key carries
// max = -inf and weighs nothing (its output is zero)
// (a: for the sink, the output scale and the row layout of dst; HM = H * maps)
__global__ void __launch_bounds__(128) k_cached_attention_merge(CaArgs a, const float* __restrict__ part, uint32_t dv, uint32_t splits,
                                                                uint32_t wkind) {
    pdl_enter();
    __shared__ float w[kCtMaxSplits];
    const float* P = part + (size_t)blockIdx.x * splits * (4 + dv);
    const uint32_t HM = a.H * a.maps, hm = blockIdx.x % HM;
    if (wkind) {                                       // unnormalised weights: the shares just add up
        if (threadIdx.x < splits) w[threadIdx.x] = a.out_scale;
    } else if (threadIdx.x < 32) {                            // warp 0: the shares' weights exp(m_i - M) / L
        float m0 = threadIdx.x < splits ? P[threadIdx.x * (4 + dv)] : -INFINITY, m1 = threadIdx.x + 32 < splits ? P[(threadIdx.x + 32) * (4 + dv)] : -INFINITY;
        float l0 = threadIdx.x < splits ? P[threadIdx.x * (4 + dv) + 1] : 0.0f, l1 = threadIdx.x + 32 < splits ? P[(threadIdx.x + 32) * (4 + dv) + 1] : 0.0f;
        const float M = warp_max(fmaxf(m0, m1));
        const float e0 = m0 == -INFINITY ? 0.0f : expf(m0 - M), e1 = m1 == -INFINITY ? 0.0f : expf(m1 - M);
        const float inv = ca_inv_sum(a, hm, M, warp_sum(l0 * e0 + l1 * e1)) * a.out_scale;
        if (threadIdx.x < splits) w[threadIdx.x] = e0 * inv;
        if (threadIdx.x + 32 < splits) w[threadIdx.x + 32] = e1 * inv;
    }
    __syncthreads();
    const uint32_t c = blockIdx.y * 128 + threadIdx.x;
    if (c >= dv) return;
    float acc = 0.0f;
#pragma unroll 4
    for (uint32_t i = 0; i < splits; i++) acc = fmaf(P[i * (4 + dv) + 4 + c], w[i], acc);
    a.dst[(size_t)(blockIdx.x / HM) * a.dst_rs + (size_t)hm * dv + c] = acc;
}

// Few query rows (decoding: tokens x heads of a key group <= 16): what bounds the step is the latency of pulling the cache,
// so a CTA takes one share of the keys, 32 at a time with WHOLE rows in shared memory — one round of loads per 32 keys instead
// of one per 64-wide slice — and the shares are merged afterwards.  Scores: the 16 x 32 (row, key) pairs are covered by 32
// threads holding 4 x 4 pairs each (rows rg + 4 r, keys kg + 8 c: conflict-free 16-byte reads of padded rows), and the eight
// warps split the key dimension; their partial dot products meet in shared memory.  Then thread (row, kq) of 16 x 16 owns
// keys kq and kq + 16 of its row, and the 16 threads of a row keep the row's running (max, sum) in step through half-warp
// shuffles; for the weighted sum thread t owns value columns t + 256 i of all rows.  Where the value row is the head of the
// key row itself (a latent that serves as both), it is not loaded twice.
constexpr int kCfRows = 16, kCfKeys = 32, kCfThreads = 256, kCfParts = kCfThreads / 32;
template <int CI>
__global__ void __launch_bounds__(kCfThreads) k_cached_attention_few(CaArgs a, uint32_t rh, uint32_t splits, float* __restrict__ part, uint32_t alias) {
    pdl_enter();
    extern __shared__ __align__(16) float sm[];
    const uint32_t KP = a.dk + 4, VP = alias ? KP : a.dv;
    float* Qs = sm;                                    // [16][dk + 4]
    float* Ks = Qs + kCfRows * KP;                     // [32][dk + 4]
    float* Sp = Ks + kCfKeys * KP;                     // [8][16][32] partial scores of the eight slices of the key dimension
    float* Ss = Sp + kCfParts * kCfRows * kCfKeys;     // [16][32] probabilities
    float* Al = Ss + kCfRows * kCfKeys;                // [16] rescale of the running sums (at the end: 1 / sum)
    float* Vs = alias ? Ks : Al + kCfRows;             // [32][dv]
    const uint32_t tid = threadIdx.x, row = tid >> 4, kq = tid & 15;
    const uint32_t warp = tid >> 5, rg = (tid & 31) >> 3, kg = tid & 7;
    const uint32_t gm = blockIdx.x, g = gm / a.maps, m = gm % a.maps;
    const uint32_t pos0 = (uint32_t)ctl_word(a.ctl, ZG_CTL_POS), slot = ca_slot(a);
    const uint32_t total = a.T * rh, p_max = pos0 + a.T - 1;
    const uint32_t k_lo = mask_low(pos0, a.kind, a.size);
    const uint32_t n_keys = p_max - k_lo + 1, per = (n_keys + splits - 1) / splits;
    const uint32_t k_begin = k_lo + blockIdx.y * per, k_end = min(p_max + 1, k_begin + per);
    const float* kbase = a.kc + (size_t)slot * a.R * a.kw + a.k_off + (size_t)gm * a.dk;
    const float* vbase = a.vc + (size_t)slot * a.R * a.vw + a.v_off + (size_t)g * a.dv;
    const bool ok = row < total;
    const uint32_t p_r = pos0 + (ok ? row / rh : 0), lo_r = mask_low(p_r, a.kind, a.size);
    const float* tab_r = a.tab ? a.tab + (size_t)((g * rh + (ok ? row % rh : 0)) * a.maps + m) * a.tab_rs : nullptr;
    const uint32_t dk4 = a.dk / 4, dv4 = a.dv / 4;
    const uint32_t chunk4 = (dk4 + kCfParts - 1) / kCfParts, d_begin = 4 * min(dk4, warp * chunk4), d_end = 4 * min(dk4, (warp + 1) * chunk4);
    for (uint32_t i = tid; i < kCfRows * dk4; i += kCfThreads) {     // rows past the step's are zero: their scores are never used
        const uint32_t r = i / dk4, c4 = i % dk4;
        copy16(Qs + r * KP + 4 * c4, r < total ? a.q + (size_t)(r / rh) * a.q_rs + a.q_off + (size_t)((g * rh + r % rh) * a.maps + m) * a.dk + 4 * c4 : a.q, r < total);
    }
    float acc[kCfRows][CI];
#pragma unroll
    for (int r = 0; r < kCfRows; r++)
#pragma unroll
        for (int i = 0; i < CI; i++) acc[r][i] = 0.0f;
    float m_run = -INFINITY, l_run = 0.0f;
    for (uint32_t s0 = k_begin; s0 < k_end; s0 += kCfKeys) {
        const uint32_t nk = min((uint32_t)kCfKeys, k_end - s0);
        __syncthreads();                               // the previous keys' readers are done
        for (uint32_t i = tid; i < kCfKeys * dk4; i += kCfThreads) {
            const uint32_t kk = i / dk4, c4 = i % dk4;
            copy16(Ks + kk * KP + 4 * c4, kk < nk ? kbase + (size_t)((s0 + kk) % a.R) * a.kw + 4 * c4 : kbase, kk < nk);
        }
        if (!alias)
            for (uint32_t i = tid; i < nk * dv4; i += kCfThreads) {
                const uint32_t kk = i / dv4, c4 = i % dv4;
                copy16(Vs + kk * VP + 4 * c4, vbase + (size_t)((s0 + kk) % a.R) * a.vw + 4 * c4, true);
            }
        asm volatile("cp.async.commit_group;" ::: "memory");   // every load of the share is in flight at once: one round trip
        asm volatile("cp.async.wait_group 0;" ::: "memory");
        __syncthreads();
        {
            float sc[4][4];
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) sc[r][c] = 0.0f;
            for (uint32_t d = d_begin; d < d_end; d += 4) {
                float4 qa[4], ka[4];
#pragma unroll
                for (int r = 0; r < 4; r++) qa[r] = *reinterpret_cast<const float4*>(Qs + (rg + 4 * r) * KP + d);
#pragma unroll
                for (int c = 0; c < 4; c++) ka[c] = *reinterpret_cast<const float4*>(Ks + (kg + 8 * c) * KP + d);
#pragma unroll
                for (int r = 0; r < 4; r++)
#pragma unroll
                    for (int c = 0; c < 4; c++) {
                        sc[r][c] = fmaf(qa[r].x, ka[c].x, sc[r][c]); sc[r][c] = fmaf(qa[r].y, ka[c].y, sc[r][c]);
                        sc[r][c] = fmaf(qa[r].z, ka[c].z, sc[r][c]); sc[r][c] = fmaf(qa[r].w, ka[c].w, sc[r][c]);
                    }
            }
#pragma unroll
            for (int r = 0; r < 4; r++)
#pragma unroll
                for (int c = 0; c < 4; c++) Sp[(warp * kCfRows + rg + 4 * r) * kCfKeys + kg + 8 * c] = sc[r][c];
        }
        __syncthreads();
        float sv[2];
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const uint32_t kk = kq + 16 * u, j = s0 + kk;
            float d = 0.0f;
#pragma unroll
            for (int w = 0; w < kCfParts; w++) d += Sp[(w * kCfRows + row) * kCfKeys + kk];
            const bool seen = ok && kk < nk && j <= p_r && j >= lo_r;
            sv[u] = seen ? ca_score(a, d) : -INFINITY;
            if (seen && tab_r) sv[u] += tab_r[p_r - j];
        }
        float rmax = fmaxf(sv[0], sv[1]);
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) rmax = fmaxf(rmax, __shfl_xor_sync(0xffffffffu, rmax, off));
        const float new_m = a.wkind ? 0.0f : fmaxf(m_run, rmax);
        const float alpha = a.wkind ? 1.0f : (m_run == -INFINITY ? (new_m == -INFINITY ? 1.0f : 0.0f) : expf(m_run - new_m));
        float rsum = 0.0f;
#pragma unroll
        for (int u = 0; u < 2; u++) {
            const float pv = sv[u] == -INFINITY ? 0.0f : (a.wkind ? ca_sigmoid(sv[u]) : expf(sv[u] - new_m));
            Ss[row * kCfKeys + kq + 16 * u] = pv;
            rsum += pv;
        }
#pragma unroll
        for (int off = 8; off > 0; off >>= 1) rsum += __shfl_xor_sync(0xffffffffu, rsum, off);
        l_run = l_run * alpha + rsum;
        m_run = new_m;
        if (kq == 0) Al[row] = alpha;
        __syncthreads();
#pragma unroll
        for (int r = 0; r < kCfRows; r++) {
            const float al = Al[r];
#pragma unroll
            for (int i = 0; i < CI; i++) acc[r][i] *= al;
        }
        for (uint32_t kk = 0; kk < nk; kk += 4) {      // four keys per trip: the probabilities are read as float4s
            float v[4][CI];
#pragma unroll
            for (int u = 0; u < 4; u++)
#pragma unroll
                for (int i = 0; i < CI; i++) { const uint32_t c = tid + kCfThreads * i; v[u][i] = (c < a.dv && kk + u < nk) ? Vs[(kk + u) * VP + c] : 0.0f; }
#pragma unroll
            for (int r = 0; r < kCfRows; r++) {
                const float4 pr = *reinterpret_cast<const float4*>(Ss + r * kCfKeys + kk);
#pragma unroll
                for (int i = 0; i < CI; i++)
                    acc[r][i] = fmaf(pr.x, v[0][i], fmaf(pr.y, v[1][i], fmaf(pr.z, v[2][i], fmaf(pr.w, v[3][i], acc[r][i]))));
            }
        }
    }
    __syncthreads();
    if (kq == 0) Al[row] = (a.wkind ? 1.0f : (l_run > 0.0f ? ca_inv_sum(a, (g * rh + (ok ? row % rh : 0)) * a.maps + m, m_run, l_run) : 0.0f)) * a.out_scale;
    if (splits > 1 && kq == 0 && ok) {
        float* mine = part + (((size_t)(row / rh) * a.H * a.maps + (g * rh + row % rh) * a.maps + m) * splits + blockIdx.y) * (4 + a.dv);
        mine[0] = m_run; mine[1] = l_run;
    }
    __syncthreads();
#pragma unroll
    for (int r = 0; r < kCfRows; r++) {
        if ((uint32_t)r >= total) break;
        const uint32_t hm_r = (g * rh + (uint32_t)r % rh) * a.maps + m;
        const size_t item = (size_t)((uint32_t)r / rh) * a.H * a.maps + hm_r;
#pragma unroll
        for (int i = 0; i < CI; i++) {
            const uint32_t c = tid + kCfThreads * i;
            if (c >= a.dv) continue;
            if (splits == 1) a.dst[(size_t)((uint32_t)r / rh) * a.dst_rs + (size_t)hm_r * a.dv + c] = acc[r][i] * Al[r];
            else part[(item * splits + blockIdx.y) * (4 + a.dv) + 4 + c] = acc[r][i];
        }
    }
}
static size_t cf_smem(uint32_t dk, uint32_t dv, bool alias) {
    return ((size_t)(kCfRows + kCfKeys) * (dk + 4) + (size_t)(kCfParts + 1) * kCfRows * kCfKeys + kCfRows + (alias ? 0 : (size_t)kCfKeys * dv)) * sizeof(float);
}
static bool cf_alias(const ZgSeqOp& s) {   // the value row is the head of the key row (one key head, one map, same cache and column)
    return s.buf[2] == s.buf[3] && s.off[1] == s.off[2] && s.n[2] == 1 && s.n[3] == 1 && s.n[5] <= s.n[4] && s.n[7] == s.n[8];
}
template <int OC>
static void launch_cached_attention_tiled(const CaArgs& a, uint32_t splits, float* part, cudaStream_t st) {
    constexpr int DV = 16 * OC;
    const size_t smem = ((size_t)(a.dk <= (uint32_t)kCtDS ? 1 : 2) * kCtBQ * kCtDS + (size_t)2 * kCtBK * (kCtDS + 4) + (size_t)kCtBQ * (kCtBK + 4) + (size_t)kCtBK * DV) * sizeof(float);
    static size_t most = 0;
    if (smem > most) { cudaFuncSetAttribute(k_cached_attention_tiled<OC>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); most = smem; }
    const uint32_t rh = a.H / a.G, n_tiles = (a.T * rh + kCtBQ - 1) / kCtBQ, n_vs = (a.dv + DV - 1) / DV;
    launch_pdl(k_cached_attention_tiled<OC>, dim3(n_tiles, a.G * a.maps * n_vs, splits), dim3(kCtThreads), smem, st, a, rh, n_tiles, splits, part);
}
static bool ca_aligned(const ZgSeqOp& s) {
    return s.n[4] % 4 == 0 && s.n[5] % 4 == 0 && s.n[6] % 4 == 0 && s.n[7] % 4 == 0 && s.n[8] % 4 == 0 && s.off[0] % 4 == 0 && s.off[1] % 4 == 0 && s.off[2] % 4 == 0;
}
static bool ca_few(const ZgSeqOp& s) {
    return ca_aligned(s) && s.n[0] * (s.n[1] / s.n[2]) <= (uint32_t)kCfRows && cf_smem(s.n[4], s.n[5], cf_alias(s)) <= 200 * 1024;
}
// key shares per row tile: few CTAs and a long cache (decoding) spread over more of them
static uint32_t ca_splits(const ZgSeqOp& s) {
    if (!ca_aligned(s)) return 1;
    if (ca_few(s)) {
        const uint32_t reach = s.off[3] ? min(s.n[9], s.off[4] + s.n[0]) : s.n[9];
        const uint32_t S = (reach + kCfKeys - 1) / kCfKeys;
        return S < 2 ? 1 : (S > (uint32_t)kCtMaxSplits ? (uint32_t)kCtMaxSplits : S);
    }
    const uint32_t rh = s.n[1] / s.n[2], n_tiles = (s.n[0] * rh + kCtBQ - 1) / kCtBQ, dvs = s.n[5] > 256 ? 512 : (s.n[5] > 128 ? 256 : 128);
    const uint32_t ctas = n_tiles * s.n[2] * s.n[3] * ((s.n[5] + dvs - 1) / dvs);
    const uint32_t reach = s.off[3] ? min(s.n[9], s.off[4] + s.n[0]) : s.n[9];     // keys a row can see at most
    uint32_t S = 160 / (ctas ? ctas : 1), most = reach / kCtMinShare;
    if (S > most) S = most;
    return S < 2 ? 1 : (S > (uint32_t)kCtMaxSplits ? (uint32_t)kCtMaxSplits : S);
}

// ── MAP_COMBINE: one warp per (token, head) ──────────────────────────────────────────────────────────────────────
__global__ void k_map_combine(float* __restrict__ dst, const float* __restrict__ src, uint32_t rows, uint32_t dv, float lambda, float eps, float out_scale) {
    pdl_enter();
    const uint32_t row = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (row >= rows) return;
    const float* a1 = src + (size_t)row * 2 * dv;
    const float* a2 = a1 + dv;
    float q = 0.0f;
    for (uint32_t c = lane; c < dv; c += 32) { const float o = fmaf(-lambda, a2[c], a1[c]); q = fmaf(o, o, q); }
    const float inv = out_scale / sqrtf(warp_sum(q) / (float)dv + eps);
    for (uint32_t c = lane; c < dv; c += 32) dst[(size_t)row * dv + c] = fmaf(-lambda, a2[c], a1[c]) * inv;
}

// ── GATE ─────────────────────────────────────────────────────────────────────────────────────────────────────────
__global__ void k_gate(float* __restrict__ dst, const float* __restrict__ gate, uint32_t T, uint32_t cols, uint32_t group, uint32_t gate_rs,
                       uint32_t gate_off, uint32_t dst_rs) {
    pdl_enter();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= (size_t)T * cols) return;
    const uint32_t t = (uint32_t)(e / cols), c = (uint32_t)(e % cols);
    dst[(size_t)t * dst_rs + c] *= sigmoidf_(gate[(size_t)t * gate_rs + gate_off + c / group]);
}

// ── HEAD_LINEAR ──────────────────────────────────────────────────────────────────────────────────────────────────
struct HlArgs {
    float* dst; const float* src; const float* gate;   // gate: output (h, n) of row m is multiplied by sigmoid(gate[m, (h N + n) / group])
    uint32_t T, H, N, K, src_hs, src_rs, dst_hs, dst_rs, gate_rs, gate_group;
};
__device__ __forceinline__ float hl_gated(const HlArgs& a, float v, uint32_t m, uint32_t h, uint32_t n) {
    return a.gate ? v * sigmoidf_(a.gate[(size_t)m * a.gate_rs + (h * a.N + n) / a.gate_group]) : v;
}
constexpr int kHlRows = 8;
// few rows: one warp per (head, output), the weight row streamed once for all rows; 16-byte weight loads (VEC) when the rows
// and the head's slices of the input start on 16-byte boundaries and K is a whole number of them
template <typename WT, bool VEC>
__global__ void k_head_linear_rows(HlArgs a, const WT* __restrict__ W) {
    pdl_enter();
    const uint32_t n = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31, h = blockIdx.y;
    if (n >= a.N) return;
    const WT* w = W + ((size_t)h * a.N + n) * a.K;
    const float* x = a.src + (size_t)h * a.src_hs;
    float acc[kHlRows];
#pragma unroll
    for (int m = 0; m < kHlRows; m++) acc[m] = 0.0f;
    if (VEC) {
        constexpr int V = WVec<WT>::n;
        for (uint32_t k = lane * V; k < a.K; k += 32 * V) {
            float wv[V];
            wld_vec<WT>(w + k, wv);
#pragma unroll
            for (int m = 0; m < kHlRows; m++) {
                if (m < (int)a.T) {
                    const float4* xv = reinterpret_cast<const float4*>(x + (size_t)m * a.src_rs + k);
#pragma unroll
                    for (int i = 0; i < V / 4; i++) {
                        const float4 q = xv[i];
                        acc[m] = fmaf(q.x, wv[4 * i], fmaf(q.y, wv[4 * i + 1], fmaf(q.z, wv[4 * i + 2], fmaf(q.w, wv[4 * i + 3], acc[m]))));
                    }
                }
            }
        }
    } else {
        for (uint32_t k = lane; k < a.K; k += 32) {
            const float wv = wld(w, k);
#pragma unroll
            for (int m = 0; m < kHlRows; m++)
                if (m < (int)a.T) acc[m] = fmaf(x[(size_t)m * a.src_rs + k], wv, acc[m]);
        }
    }
#pragma unroll
    for (int m = 0; m < kHlRows; m++) {
        if (m < (int)a.T) {
            const float s = warp_sum(acc[m]);
            if (lane == 0) a.dst[(size_t)m * a.dst_rs + (size_t)h * a.dst_hs + n] = hl_gated(a, s, m, h, n);
        }
    }
}
// many rows, exact f32: 64 x 64 tile of one head, 16-deep k slices, 4 x 4 outputs per thread
constexpr int kHlTM = 64, kHlTN = 64, kHlTK = 16;
template <typename WT>
__global__ void __launch_bounds__(256) k_head_linear_tile(HlArgs a, const WT* __restrict__ W) {
    __shared__ float As[kHlTK][kHlTM + 4];
    __shared__ float Ws[kHlTK][kHlTN + 4];
    const uint32_t h = blockIdx.z, m0 = blockIdx.y * kHlTM, n0 = blockIdx.x * kHlTN;
    const uint32_t tx = threadIdx.x & 15, ty = threadIdx.x >> 4;
    const float* src = a.src + (size_t)h * a.src_hs;
    const WT* Wh = W + (size_t)h * a.N * a.K;
    float acc[4][4] = {};
    for (uint32_t k0 = 0; k0 < a.K; k0 += kHlTK) {
        for (uint32_t e = threadIdx.x; e < kHlTM * kHlTK; e += 256) {
            const uint32_t r = e / kHlTK, kk = e % kHlTK;
            const uint32_t m = m0 + r, k = k0 + kk, n = n0 + r;
            As[kk][r] = (m < a.T && k < a.K) ? src[(size_t)m * a.src_rs + k] : 0.0f;
            Ws[kk][r] = (n < a.N && k < a.K) ? wld(Wh, (size_t)n * a.K + k) : 0.0f;
        }
        __syncthreads();
#pragma unroll
        for (int kk = 0; kk < kHlTK; kk++) {
            float x[4], w[4];
#pragma unroll
            for (int i = 0; i < 4; i++) { x[i] = As[kk][ty * 4 + i]; w[i] = Ws[kk][tx * 4 + i]; }
#pragma unroll
            for (int i = 0; i < 4; i++)
#pragma unroll
                for (int j = 0; j < 4; j++) acc[i][j] = fmaf(x[i], w[j], acc[i][j]);
        }
        __syncthreads();
    }
#pragma unroll
    for (int i = 0; i < 4; i++) {
        const uint32_t m = m0 + ty * 4 + i;
        if (m >= a.T) continue;
#pragma unroll
        for (int j = 0; j < 4; j++) {
            const uint32_t n = n0 + tx * 4 + j;
            if (n < a.N) a.dst[(size_t)m * a.dst_rs + (size_t)h * a.dst_hs + n] = hl_gated(a, acc[i][j], m, h, n);
        }
    }
}

// ── POLY_NORM: one CTA per row ───────────────────────────────────────────────────────────────────────────────────
template <typename WT>
__global__ void k_poly_norm(float* dst, const float* src, const WT* __restrict__ coeff, uint32_t cols, float eps) {
    pdl_enter();
    __shared__ float sh[32];
    const float* z = src + (size_t)blockIdx.x * cols;
    float s2 = 0.0f, s4 = 0.0f, s6 = 0.0f;
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = z[c], v2 = v * v, v3 = v2 * v;
        s2 = fmaf(v, v, s2); s4 = fmaf(v2, v2, s4); s6 = fmaf(v3, v3, s6);
    }
    const float n = (float)cols;
    const float i1 = wld(coeff, 0) / sqrtf(block_sum(s2, sh) / n + eps);
    const float i2 = wld(coeff, 1) / sqrtf(block_sum(s4, sh) / n + eps);
    const float i3 = wld(coeff, 2) / sqrtf(block_sum(s6, sh) / n + eps);
    const float e = wld(coeff, 3);
    float* out = dst + (size_t)blockIdx.x * cols;
    for (uint32_t c = threadIdx.x; c < cols; c += blockDim.x) {
        const float v = z[c], v2 = v * v;
        out[c] = fmaf(i1, v, fmaf(i2, v2, fmaf(i3, v2 * v, e)));
    }
}

}  // namespace

bool zg_mix_op_valid(const ZgOp& op, const size_t* elems, size_t n_bufs, char* why, size_t why_n) {
    const ZgSeqOp& s = op.u.seq;
    auto fail = [&](const char* m) { snprintf(why, why_n, "%s", m); return false; };
    auto have = [&](int i) { return s.buf[i] != ZG_NO_BUF && s.buf[i] < n_bufs; };
    auto fits = [&](int i, size_t off, size_t n) { return have(i) && off + n <= elems[s.buf[i]]; };
    auto wfits = [&](int i, uint32_t wdt, size_t off, size_t n) { return wdt <= ZG_W_BF16 && have(i) && (wdt == ZG_W_BF16 ? (off + n + 1) / 2 : off + n) <= elems[s.buf[i]]; };
    switch (op.tag) {
        case ZG_OP_TOKEN_SHIFT: {
            const size_t T = s.n[0], D = s.n[1];
            if (!T || !D) return fail("token_shift: shape");
            if (!fits(0, 0, T * D) || !fits(1, 0, T * D) || !wfits(2, s.n[2], s.off[0], D) || !have(3) || elems[s.buf[3]] < D || !fits(4, 0, ZG_CTL_IDS))
                return fail("token_shift: extent");
            if (s.buf[0] == s.buf[1]) return fail("token_shift: in place");
            return true;
        }
        case ZG_OP_DEPTH_MIX: {
            const size_t n = s.n[0], terms = s.n[1], stride = s.n[2];
            if (!n || !terms || stride < n) return fail("depth_mix: shape");
            if (!fits(0, 0, n) || !fits(1, 0, (terms - 1) * stride + n) || !wfits(2, s.n[3], s.off[0], terms)) return fail("depth_mix: extent");
            if (s.buf[0] == s.buf[1]) return fail("depth_mix: in place");
            return true;
        }
        case ZG_OP_ROTARY: {
            const size_t T = s.n[0], heads = s.n[1], hs = s.n[2], rs = s.n[3], dims = s.n[4];
            if (!T || !heads || !dims || dims % 2 || hs < dims || s.n[5] > 1 || (s.buf[3] == ZG_NO_BUF && !(s.f[0] > 0.0f))) return fail("rotary: shape");
            if (s.buf[3] != ZG_NO_BUF && !fits(3, s.off[2], dims / 2)) return fail("rotary: frequency table");
            if (s.off[0] + (heads - 1) * hs + dims > rs) return fail("rotary: columns");
            if (!fits(0, 0, (T - 1) * rs + s.off[0] + (heads - 1) * hs + dims) || !fits(1, 0, ZG_CTL_IDS)) return fail("rotary: extent");
            if (s.buf[2] != ZG_NO_BUF) {
                const size_t shs = s.n[6], srs = s.n[7];
                if (shs < dims || s.off[1] + (heads - 1) * shs + dims > srs || !fits(2, 0, (T - 1) * srs + s.off[1] + (heads - 1) * shs + dims) || s.buf[2] == s.buf[0])
                    return fail("rotary: source");
            }
            return true;
        }
        case ZG_OP_CACHE_APPEND: {
            const size_t T = s.n[0], cols = s.n[1], srs = s.n[2], width = s.n[3], R = s.n[4];
            const size_t normed = s.n[5], rot = s.n[6];
            if (!T || !cols || R < T || s.off[0] + cols > srs || s.off[1] + cols > width || normed + rot > cols || rot % 2 || s.n[8] > 1) return fail("cache_append: shape");
            if (!have(0) || elems[s.buf[0]] < R * width || !fits(1, 0, (T - 1) * srs + s.off[0] + cols) || !fits(2, 0, ZG_CTL_IDS)) return fail("cache_append: extent");
            if (normed && s.n[9] && normed % s.n[9]) return fail("cache_append: norm groups");
            if (normed && !wfits(3, s.n[7], s.off[2], s.n[9] ? s.n[9] : normed)) return fail("cache_append: norm weight");
            if (rot && !(s.f[1] > 0.0f)) return fail("cache_append: rotary base");
            if (s.n[10]) {     // rotary inside every normed head, before its norm
                if (!normed || !s.n[9] || rot || s.n[10] % 2 || s.n[10] > s.n[9]) return fail("cache_append: head rotary");
                if (s.buf[4] != ZG_NO_BUF ? !fits(4, s.off[7], s.n[10] / 2) : !(s.f[1] > 0.0f)) return fail("cache_append: head rotary frequencies");
            }
            if (s.off[5]) {    // query heads normed in place in the source rows
                const size_t qh = s.off[5], hd = s.n[9];
                if (!normed || !hd || s.off[3] + qh * hd > srs || !fits(1, 0, (T - 1) * srs + s.off[3] + qh * hd) || !wfits(3, s.n[7], s.off[4], hd)) return fail("cache_append: query heads");
                if (s.off[3] < s.off[0] + cols && s.off[0] < s.off[3] + qh * hd) return fail("cache_append: query heads overlap the appended columns");
            }
            return true;
        }
        case ZG_OP_CACHED_ATTENTION: {
            const size_t T = s.n[0], H = s.n[1], G = s.n[2], maps = s.n[3], dk = s.n[4], dv = s.n[5], qrs = s.n[6], kw = s.n[7], vw = s.n[8], R = s.n[9];
            const uint32_t kind = s.off[3], size = s.off[4];
            if (!T || !H || !G || H % G || !maps || !dk || !dv || dv > kCaMaxDv || kind > 2 || (kind && !size)) return fail("cached_attention: shape");
            if (R < T) return fail("cached_attention: cache rows");   // the caller sizes R for what the mask reaches and bounds the positions
            if (s.off[0] + H * maps * dk > qrs || s.off[1] + G * maps * dk > kw || s.off[2] + G * dv > vw) return fail("cached_attention: columns");
            const size_t drs = s.n[10] ? s.n[10] : H * maps * dv;
            if (s.n[11] + H * maps * dv > drs || s.f[1] < 0.0f || s.n[13] > 1 || s.n[14] > 1) return fail("cached_attention: destination columns, cap or output scale");
            if (s.buf[6] != ZG_NO_BUF && (s.off[5] || !wfits(6, s.n[12], s.off[7], H * maps))) return fail("cached_attention: sinks");
            if (!fits(0, 0, (T - 1) * drs + s.n[11] + H * maps * dv) || !fits(1, 0, (T - 1) * qrs + s.off[0] + H * maps * dk) || !have(2) || elems[s.buf[2]] < R * kw || !have(3) ||
                elems[s.buf[3]] < R * vw || !fits(4, 0, ZG_CTL_IDS))
                return fail("cached_attention: extent");
            if (s.buf[0] == s.buf[1]) return fail("cached_attention: in place");
            if (s.off[5] > 1) return fail("cached_attention: weights");
            if (s.buf[5] != ZG_NO_BUF) {               // the table must cover every distance the mask lets a query reach
                const size_t reach = kind == 0 ? R : (size < R ? size : R);
                if (s.off[6] < reach || !fits(5, 0, H * maps * (size_t)s.off[6])) return fail("cached_attention: score table");
            }
            return true;
        }
        case ZG_OP_MAP_COMBINE: {
            const size_t rows = s.n[0], dv = s.n[1];
            if (!rows || !dv) return fail("map_combine: shape");
            if (!fits(0, 0, rows * dv) || !fits(1, 0, rows * 2 * dv) || s.buf[0] == s.buf[1]) return fail("map_combine: extent");
            return true;
        }
        case ZG_OP_GATE: {
            const size_t T = s.n[0], cols = s.n[1], group = s.n[2], grs = s.n[3], drs = s.n[4];
            if (!T || !cols || !group || cols % group || drs < cols || s.off[0] + cols / group > grs) return fail("gate: shape");
            if (!fits(0, 0, (T - 1) * drs + cols) || !fits(1, 0, (T - 1) * grs + s.off[0] + cols / group)) return fail("gate: extent");
            return true;
        }
        case ZG_OP_HEAD_LINEAR: {
            const size_t T = s.n[0], H = s.n[1], N = s.n[2], K = s.n[3], shs = s.n[4], srs = s.n[5], dhs = s.n[6], drs = s.n[7];
            if (!T || !H || !N || !K || shs < K || dhs < N || s.off[1] + (H - 1) * shs + K > srs || s.off[2] + (H - 1) * dhs + N > drs) return fail("head_linear: shape");
            if (!fits(0, 0, (T - 1) * drs + s.off[2] + (H - 1) * dhs + N) || !fits(1, 0, (T - 1) * srs + s.off[1] + (H - 1) * shs + K) || !wfits(2, s.n[8], s.off[0], H * N * K))
                return fail("head_linear: extent");
            if (s.buf[0] == s.buf[1]) return fail("head_linear: in place");
            if (s.buf[3] != ZG_NO_BUF) {
                const size_t group = s.n[9], grs = s.off[4];
                if (!group || (H * N) % group || s.off[3] + H * N / group > grs || !fits(3, 0, (T - 1) * grs + s.off[3] + H * N / group) || s.buf[3] == s.buf[0]) return fail("head_linear: gate");
            }
            return true;
        }
        case ZG_OP_POLY_NORM: {
            const size_t n = (size_t)s.n[0] * s.n[1];
            if (!n) return fail("poly_norm: shape");
            if (!fits(0, 0, n) || !fits(1, 0, n) || !wfits(2, s.n[2], s.off[0], 4)) return fail("poly_norm: extent");
            return true;
        }
        default: return fail("not a sequence op");
    }
}

uint32_t zg_mix_op_writes(uint32_t tag) {
    if (tag == ZG_OP_CACHE_APPEND) return 1u | (1u << 1);   // the source rows too: query heads may be normed in place
    return tag == ZG_OP_TOKEN_SHIFT ? (1u | (1u << 3)) : 1u;
}

size_t zg_mix_op_scratch_elems(const ZgOp& op) {
    if (op.tag != ZG_OP_CACHED_ATTENTION) return 0;
    const ZgSeqOp& s = op.u.seq;
    const uint32_t S = ca_splits(s);
    return S > 1 ? (size_t)s.n[0] * s.n[1] * s.n[3] * S * (4 + s.n[5]) : 0;
}

bool zg_launch_mix_op(const ZgOp& op, float* const* bufs, float* scratch, cudaStream_t st) {
    (void)scratch;
    const ZgSeqOp& s = op.u.seq;
    switch (op.tag) {
        case ZG_OP_TOKEN_SHIFT: {
            const size_t n = (size_t)s.n[0] * s.n[1];
            ZG_SEQ_WDT(s.n[2], launch_pdl(k_token_shift<WT>, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], wptr<WT>(bufs, s.buf[2], s.off[0]),
                                          bufs[s.buf[3]], bufs[s.buf[4]], s.n[0], s.n[1]));
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_DEPTH_MIX:
            ZG_SEQ_WDT(s.n[3], launch_pdl(k_depth_mix<WT>, dim3((s.n[0] + 255) / 256), dim3(256), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], wptr<WT>(bufs, s.buf[2], s.off[0]), s.n[0], s.n[1], s.n[2]));
            ZG_SEQ_CHECK();
            return true;
        case ZG_OP_ROTARY: {
            const size_t n = (size_t)s.n[0] * s.n[1] * (s.n[4] / 2);
            float* x = bufs[s.buf[0]] + s.off[0];
            const bool sep = s.buf[2] != ZG_NO_BUF;
            launch_pdl(k_rotary, dim3((unsigned)((n + 127) / 128)), dim3(128), 0, st, x, sep ? bufs[s.buf[2]] + s.off[1] : x, bufs[s.buf[1]], s.n[0], s.n[1], s.n[2], s.n[3], s.n[4], s.n[5],
                       sep ? s.n[6] : s.n[2], sep ? s.n[7] : s.n[3], s.f[0], s.buf[3] != ZG_NO_BUF ? (const float*)(bufs[s.buf[3]] + s.off[2]) : (const float*)nullptr);
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_CACHE_APPEND:
            ZG_SEQ_WDT(s.n[5] ? s.n[7] : ZG_W_F32, launch_pdl(k_cache_append<WT>, dim3(s.n[0]), dim3(s.off[5] ? 256 : 128), (size_t)s.n[10] * sizeof(float), st, bufs[s.buf[0]] + s.off[1], bufs[s.buf[1]] + s.off[0], bufs[s.buf[2]],
                                                             s.n[5] ? wptr<WT>(bufs, s.buf[3], s.off[2]) : nullptr, s.n[1], s.n[2], s.n[3], s.n[4], s.n[5], s.n[6], s.n[8], s.f[0], s.f[1], s.n[9],
                                                             s.off[5] ? bufs[s.buf[1]] + s.off[3] : nullptr, s.off[5] ? wptr<WT>(bufs, s.buf[3], s.off[4]) : nullptr, s.off[5], s.off[6], s.f[2],
                                                             s.n[10], s.n[10] && s.buf[4] != ZG_NO_BUF ? (const float*)(bufs[s.buf[4]] + s.off[7]) : (const float*)nullptr));
            ZG_SEQ_CHECK();
            return true;
        case ZG_OP_CACHED_ATTENTION: {
            CaArgs a;
            a.dst = bufs[s.buf[0]]; a.q = bufs[s.buf[1]]; a.kc = bufs[s.buf[2]]; a.vc = bufs[s.buf[3]]; a.ctl = bufs[s.buf[4]];
            a.T = s.n[0]; a.H = s.n[1]; a.G = s.n[2]; a.maps = s.n[3]; a.dk = s.n[4]; a.dv = s.n[5]; a.q_rs = s.n[6]; a.q_off = s.off[0];
            a.kw = s.n[7]; a.k_off = s.off[1]; a.vw = s.n[8]; a.v_off = s.off[2]; a.R = s.n[9]; a.kind = s.off[3]; a.size = s.off[4]; a.scale = s.f[0];
            a.tab = s.buf[5] != ZG_NO_BUF ? bufs[s.buf[5]] : nullptr; a.tab_rs = s.off[6]; a.wkind = s.off[5];
            a.cap = s.f[1]; a.out_scale = s.n[13] ? s.f[2] : 1.0f; a.dst_rs = s.n[10] ? s.n[10] : a.H * a.maps * a.dv; a.dst += s.n[11];
            a.sink = nullptr; a.sink_bf16 = s.n[12] == ZG_W_BF16; a.unslotted = s.n[14];
            if (s.buf[6] != ZG_NO_BUF) a.sink = a.sink_bf16 ? (const void*)wptr<bf16>(bufs, s.buf[6], s.off[7]) : (const void*)wptr<float>(bufs, s.buf[6], s.off[7]);
            const bool aligned = ca_aligned(s) && ((reinterpret_cast<uintptr_t>(a.q) | reinterpret_cast<uintptr_t>(a.kc) | reinterpret_cast<uintptr_t>(a.vc)) & 15) == 0;
            if (aligned && ca_few(s)) {
                const uint32_t S = scratch ? ca_splits(s) : 1, alias = cf_alias(s) ? 1u : 0u;
                float* part = S > 1 ? scratch : nullptr;
                const size_t smem = cf_smem(a.dk, a.dv, alias != 0);
                const dim3 grid(a.G * a.maps, S);
#define ZG_CF(CI_)                                                                                                                         \
    do {                                                                                                                                   \
        static size_t most = 48 * 1024;                                                                                                    \
        if (smem > most) { cudaFuncSetAttribute(k_cached_attention_few<CI_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem); most = smem; } \
        launch_pdl(k_cached_attention_few<CI_>, grid, dim3(kCfThreads), smem, st, a, a.H / a.G, S, part, alias);                            \
    } while (0)
                if (a.dv <= 256) ZG_CF(1); else if (a.dv <= 512) ZG_CF(2); else ZG_CF(4);
#undef ZG_CF
                if (S > 1) {
                    ZG_SEQ_CHECK();
                    launch_pdl(k_cached_attention_merge, dim3(a.T * a.H * a.maps, (a.dv + 127) / 128), dim3(128), 0, st, a, (const float*)part, a.dv, S, a.wkind);
                }
            } else if (aligned) {
                const uint32_t S = scratch ? ca_splits(s) : 1;
                float* part = S > 1 ? scratch : nullptr;
                // A latent of rank <= 512 in ONE value slice takes its scores once instead of once per 256 columns, but halves the
                // number of CTAs: worth it only while they still fill the GPU one and a half times.
                static int n_sm = 0;
                if (!n_sm) { int dev = 0; cudaGetDevice(&dev); cudaDeviceGetAttribute(&n_sm, cudaDevAttrMultiProcessorCount, dev); if (n_sm <= 0) n_sm = 1; }
                const uint32_t row_ctas = ((a.T * (a.H / a.G) + kCtBQ - 1) / kCtBQ) * a.G * a.maps * S * ((a.dv + 511) / 512);
                if (a.dv > 256 && 2 * row_ctas >= 3 * (uint32_t)n_sm) launch_cached_attention_tiled<32>(a, S, part, st);
                else if (a.dv > 128) launch_cached_attention_tiled<16>(a, S, part, st);
                else switch ((a.dv + 15) / 16) {
                    case 1: launch_cached_attention_tiled<1>(a, S, part, st); break;
                    case 2: launch_cached_attention_tiled<2>(a, S, part, st); break;
                    case 3: case 4: launch_cached_attention_tiled<4>(a, S, part, st); break;
                    case 5: case 6: launch_cached_attention_tiled<6>(a, S, part, st); break;
                    default: launch_cached_attention_tiled<8>(a, S, part, st); break;
                }
                if (S > 1) {
                    ZG_SEQ_CHECK();
                    launch_pdl(k_cached_attention_merge, dim3(a.T * a.H * a.maps, (a.dv + 127) / 128), dim3(128), 0, st, a, (const float*)part, a.dv, S, a.wkind);
                }
            } else {
                const uint32_t warps = 4, items = a.T * a.H * a.maps;
                launch_pdl(k_cached_attention, dim3((items + warps - 1) / warps), dim3(warps * 32), warps * a.dk * sizeof(float), st, a);
            }
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_MAP_COMBINE:
            launch_pdl(k_map_combine, dim3((s.n[0] + 3) / 4), dim3(128), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], s.n[0], s.n[1], s.f[0], s.f[1], s.f[2]);
            ZG_SEQ_CHECK();
            return true;
        case ZG_OP_GATE: {
            const size_t n = (size_t)s.n[0] * s.n[1];
            launch_pdl(k_gate, dim3((unsigned)((n + 255) / 256)), dim3(256), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], s.n[0], s.n[1], s.n[2], s.n[3], s.off[0], s.n[4]);
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_HEAD_LINEAR: {
            HlArgs a;
            a.dst = bufs[s.buf[0]] + s.off[2]; a.src = bufs[s.buf[1]] + s.off[1];
            a.T = s.n[0]; a.H = s.n[1]; a.N = s.n[2]; a.K = s.n[3]; a.src_hs = s.n[4]; a.src_rs = s.n[5]; a.dst_hs = s.n[6]; a.dst_rs = s.n[7];
            a.gate = s.buf[3] != ZG_NO_BUF ? bufs[s.buf[3]] + s.off[3] : nullptr; a.gate_rs = s.off[4]; a.gate_group = s.n[9];
            ZG_SEQ_WDT(s.n[8], {
                const WT* W = wptr<WT>(bufs, s.buf[2], s.off[0]);
                constexpr uint32_t V = WVec<WT>::n;
                const bool vec = a.K % V == 0 && a.src_hs % 4 == 0 && a.src_rs % 4 == 0 && ((reinterpret_cast<uintptr_t>(W) | reinterpret_cast<uintptr_t>(a.src)) & 15) == 0;
                if (a.T <= (uint32_t)kHlRows && vec) launch_pdl(k_head_linear_rows<WT, true>, dim3((a.N + 7) / 8, a.H), dim3(256), 0, st, a, W);
                else if (a.T <= (uint32_t)kHlRows) launch_pdl(k_head_linear_rows<WT, false>, dim3((a.N + 7) / 8, a.H), dim3(256), 0, st, a, W);
                else k_head_linear_tile<WT><<<dim3((a.N + kHlTN - 1) / kHlTN, (a.T + kHlTM - 1) / kHlTM, a.H), 256, 0, st>>>(a, W);
            });
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_POLY_NORM:
            ZG_SEQ_WDT(s.n[2], launch_pdl(k_poly_norm<WT>, dim3(s.n[0]), dim3(256), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], wptr<WT>(bufs, s.buf[2], s.off[0]), s.n[1], s.f[0]));
            ZG_SEQ_CHECK();
            return true;
        default:
            zg_set_error("unsupported sequence op tag %u", op.tag);
            return false;
    }
}
