// Sequence-model DeviceOps ZG_OP_SSM_SCAN .. ZG_OP_RG_LRU (parameter packs in include/zgml_cuda.h): recurrent mixers
// whose decay is a scalar per head (the state-space scan of Mamba-2) or a gate per element (the minimal gated recurrent
// unit), the gated group norm that closes the former, a per-head RMS norm with a position-dependent temperature, and
// stand-alone activations.  Everything here is f32: step sizes, softplus and exponentials, decays, gates, the states and
// their read-outs, norms and positions.
#include "seq_common.cuh"

#include <math.h>

namespace {

// Walks over many tokens (SSM_SCAN, MIN_GRU from kLongWalk tokens on) are launched WITHOUT programmatic early start.  Such a
// kernel has few CTAs (one per SM or fewer) and is bound by the dependent issue of single warps.  Started early, its CTAs are
// placed while the predecessor's last wave still fills the GPU: on the few SMs that have room, several per SM, where they
// stay for the whole walk and share issue slots.  Measured on a 1024-token step of a 4-layer model at width 2048: 3.02 ms with
// the scan started early, 2.36 ms without (the scan alone: 252 us either way as a one-op program).  Single-token steps keep
// the early start: there the launch gap is what counts.
constexpr int kLongWalk = 64;

// ── SSM_SCAN ─────────────────────────────────────────────────────────────────────────────────────────────────────
// Columns of a head's state S [N, P] evolve independently given the token's B, C, decay and step size, so a head is split by
// columns over CTAs.  A thread keeps a block of 16 RQ state rows x 2 columns in registers (RQ = 1 / 2 / 4 for N <= 128 / 256 /
// 512) as PAIRS OF ROWS: a float4 of B or C read from shared memory is two such pairs as it stands, so the update
// S = a S + B (dt x) and the read-out y += S C are packed f32x2 instructions with no repacking, every B and C value serves
// two columns, and most of the read-out sum stays inside the thread.  (One column and 8 rows per thread was bound by
// shared-memory wavefronts; 4 x 4 blocks by instructions per state element: shuffles, selects and register moves.)  The NS
// threads that share two columns sit in adjacent lanes (NS a power of two <= 8); thread s owns the float4s s + NS i (i < 4 RQ)
// of the rows, so the NS lanes read consecutive float4s.  What is left of the read-out sum crosses the NS lanes in a scatter:
// after the first step a lane carries one of the two columns.
// Step sizes and decays of the head (softplus, two exponentials) are evaluated for a span of tokens at once, in parallel,
// before the walk; B, C and the CTA's x columns arrive in tiles of kSsmTile tokens through cp.async, two tiles in flight, so
// the next tile's loads run under this tile's walk; four tokens are walked per trip so that their loads and sums interleave.
// A step of many tokens in a model with few (head, column block) pairs is cut into segments walked side by side (SsmArgs::mode).
// State in memory: [H][column blocks][32 RQ][kSsmThreads], element (i, thread) — each thread's block, fully coalesced; the
// layout is private to the op (zeros mean an empty state in any layout).
constexpr int kSsmThreads = 128, kSsmTile = 16, kSsmSpan = 1024, kSsmMaxN = 512;
__host__ __device__ inline uint32_t ssm_rq(uint32_t N) { return N > 256 ? 4 : (N > 128 ? 2 : 1); }
__host__ __device__ inline uint32_t ssm_slices(uint32_t N) {
    uint32_t ns = 1;
    while (ns * 16 * ssm_rq(N) < N) ns <<= 1;
    return ns;
}
struct SsmArgs {
    float* dst; const float* xbc; const float* dtl; float* state; const float* ctl;
    uint32_t T, H, G, N, P, x_off, b_off, c_off, dt_off, xbc_rs, dt_rs, vec;
    // Segments of a long step walked side by side (the recurrence is linear in the state).  mode 0: the whole step from the carried
    // state.  mode 1: segment blockIdx.z from an EMPTY state, no read-out; leaves the state it reaches and the product of its decays.
    // mode 2: segment blockIdx.z from the state it really starts from (segment 0: the carried one), with the read-out; the last
    // segment leaves the carried state.  Between the two, k_ssm_fold turns the reached states into starting states.
    uint32_t mode, seg_len;
    float* seg_state;      // [segments - 1][state elements of one slot]
    float* seg_decay;      // [segments - 1][H]
};
// global -> shared without passing through registers, 4 or 16 bytes; `on` false writes zeros (nothing is read)
__device__ __forceinline__ void ssm_copy4(float* dst, const float* src, bool on) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = on ? 4 : 0;
    asm volatile("cp.async.ca.shared.global [%0], [%1], 4, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
__device__ __forceinline__ void ssm_copy16(float* dst, const float* src, bool on) {
    const uint32_t d = (uint32_t)__cvta_generic_to_shared(dst);
    const int n = on ? 16 : 0;
    asm volatile("cp.async.cg.shared.global [%0], [%1], 16, %2;" ::"r"(d), "l"(src), "r"(n) : "memory");
}
template <typename WT, uint32_t NS, int RQ>
__global__ void __launch_bounds__(kSsmThreads) k_ssm_scan(SsmArgs a, const WT* __restrict__ a_log, const WT* __restrict__ dt_bias, const WT* __restrict__ dskip) {
    asm volatile("griddepcontrol.wait;" ::: "memory");       // the dependent kernel is let in when the walk is over (below)
    constexpr uint32_t CPB = kSsmThreads / NS * 2, NP = NS * 16 * RQ, NI = 4 * RQ;   // columns per CTA, padded state rows, float4s of rows per thread
    extern __shared__ __align__(16) float sm[];
    constexpr uint32_t kStage = kSsmTile * (2 * NP + CPB);               // per stage: B [tile][NP], C [tile][NP], x [tile][CPB]
    float* Dt = sm + 2 * kStage;                                         // step sizes and decays of a span of tokens
    float* Dec = Dt + kSsmSpan;
    const uint32_t tid = threadIdx.x, s = tid % NS, pl = tid / NS;
    const uint32_t h = blockIdx.y, cb = blockIdx.x, g = h / (a.H / a.G);
    const uint32_t p0 = cb * CPB + pl * 2;                               // this thread's first column
    const uint32_t slot = (uint32_t)ctl_word(a.ctl, ZG_CTL_SLOT);
    const uint32_t n_cb = (a.P + CPB - 1) / CPB;
    constexpr size_t kBlock = (size_t)32 * RQ * kSsmThreads;             // state elements of one (head, column block)
    const size_t slot_elems = (size_t)a.H * n_cb * kBlock, my_block = ((size_t)h * n_cb + cb) * kBlock;
    float* st = a.state + slot * slot_elems + my_block;
    const uint32_t seg = a.mode ? blockIdx.z : 0, n_seg = a.mode ? (a.T + a.seg_len - 1) / a.seg_len : 1;
    const uint32_t t_begin = a.mode ? seg * a.seg_len : 0, t_end = a.mode ? min(a.T, t_begin + a.seg_len) : a.T;
    const float* from = a.mode == 2 && seg > 0 ? a.seg_state + (size_t)(seg - 1) * slot_elems + my_block : st;
    float2 S[NI][2][2];                                                  // [float4 of rows][pair of rows in it][column]
#pragma unroll
    for (int i = 0; i < 16 * RQ; i++) {
        S[i / 4][(i / 2) % 2][i % 2].x = a.mode == 1 ? 0.0f : from[(2 * i) * kSsmThreads + tid];
        S[i / 4][(i / 2) % 2][i % 2].y = a.mode == 1 ? 0.0f : from[(2 * i + 1) * kSsmThreads + tid];
    }
    float decay_product = 1.0f;                                          // mode 1, thread 0
    const float neg_a = -expf(wld(a_log, h)), bias = wld(dt_bias, h), dsk = wld(dskip, h);
    const float* bsrc = a.xbc + a.b_off + (size_t)g * a.N;
    const float* csrc = a.xbc + a.c_off + (size_t)g * a.N;
    const float* xsrc = a.xbc + a.x_off + (size_t)h * a.P + (size_t)cb * CPB;
    const uint32_t x_cols = min(CPB, a.P - cb * CPB);
    // which of its two columns the thread ends up with after the scattered reduction, and whether it is the one that writes it
    const bool up = NS >= 2 && (s & (NS / 2)) != 0;
    const bool writer = NS >= 2 ? (s & (NS / 2 - 1)) == 0 : true;

    auto fetch_tile = [&](uint32_t t0, uint32_t stage) {
        float* Bs = sm + stage * kStage;
        float* Cs = Bs + kSsmTile * NP;
        float* Xs = Cs + kSsmTile * NP;
        const uint32_t nt = min((uint32_t)kSsmTile, t_end - t0);
        if (a.vec) {
            for (uint32_t e = tid; e < nt * (NP / 4); e += kSsmThreads) {
                const uint32_t tt = e / (NP / 4), n = 4 * (e % (NP / 4));
                const bool on = n < a.N;
                ssm_copy16(Bs + tt * NP + n, on ? bsrc + (size_t)(t0 + tt) * a.xbc_rs + n : a.xbc, on);
                ssm_copy16(Cs + tt * NP + n, on ? csrc + (size_t)(t0 + tt) * a.xbc_rs + n : a.xbc, on);
            }
            for (uint32_t e = tid; e < nt * (CPB / 4); e += kSsmThreads) {
                const uint32_t tt = e / (CPB / 4), c = 4 * (e % (CPB / 4));
                const bool on = c < x_cols;
                ssm_copy16(Xs + tt * CPB + c, on ? xsrc + (size_t)(t0 + tt) * a.xbc_rs + c : a.xbc, on);
            }
            return;
        }
        for (uint32_t e = tid; e < nt * NP; e += kSsmThreads) {
            const uint32_t tt = e / NP, n = e % NP;
            const bool on = n < a.N;
            ssm_copy4(Bs + e, on ? bsrc + (size_t)(t0 + tt) * a.xbc_rs + n : a.xbc, on);
            ssm_copy4(Cs + e, on ? csrc + (size_t)(t0 + tt) * a.xbc_rs + n : a.xbc, on);
        }
        for (uint32_t e = tid; e < nt * CPB; e += kSsmThreads) {
            const uint32_t tt = e / CPB, c = e % CPB;
            const bool on = c < x_cols;
            ssm_copy4(Xs + e, on ? xsrc + (size_t)(t0 + tt) * a.xbc_rs + c : a.xbc, on);
        }
    };
    for (uint32_t base = t_begin; base < t_end; base += kSsmSpan) {
        const uint32_t span = min((uint32_t)kSsmSpan, t_end - base);
        __syncthreads();                                   // the previous span's readers are done
        fetch_tile(base, 0);
        asm volatile("cp.async.commit_group;" ::: "memory");
        for (uint32_t t = tid; t < span; t += kSsmThreads) {
            const float dt = softplusf_(a.dtl[(size_t)(base + t) * a.dt_rs + a.dt_off + h] + bias);
            Dt[t] = dt;
            Dec[t] = expf(neg_a * dt);
        }
        for (uint32_t t0 = 0, it = 0; t0 < span; t0 += kSsmTile, it++) {
            const uint32_t stage = it & 1;
            asm volatile("cp.async.wait_group 0;" ::: "memory");
            __syncthreads();                               // tile `it` has landed for everyone, and everyone has left tile it - 1
            if (a.mode == 1 && tid == 0)
                for (uint32_t t = t0; t < min(span, t0 + kSsmTile); t++) decay_product *= Dec[t];
            if (t0 + kSsmTile < span) fetch_tile(base + t0 + kSsmTile, stage ^ 1);
            asm volatile("cp.async.commit_group;" ::: "memory");
            const float* Bs = sm + stage * kStage;
            const float* Cs = Bs + kSsmTile * NP;
            const float* Xs = Cs + kSsmTile * NP;
            const uint32_t nt = min((uint32_t)kSsmTile, span - t0);
            constexpr int U = RQ > 1 ? 2 : 4;              // tokens per trip (4: 238 us per 1024-token walk at 64 heads, 2: 252, 1: 267)
            float* out = a.dst + (size_t)(base + t0) * a.H * a.P + (size_t)h * a.P + p0;
            for (uint32_t tt = 0; tt < nt; tt += U) {
                float2 x[U], d2[U], tx[U][2], y[U][2];
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const uint32_t tu = min(tt + u, nt - 1);       // a token past the tile's end repeats the last one with decay 1 and step 0: the state stays
                    const bool live = tt + u < nt;
                    x[u] = *reinterpret_cast<const float2*>(Xs + tu * CPB + pl * 2);
                    const float dec = live ? Dec[t0 + tu] : 1.0f, dt = live ? Dt[t0 + tu] : 0.0f;
                    d2[u] = make_float2(dec, dec);
                    tx[u][0] = make_float2(dt * x[u].x, dt * x[u].x);
                    tx[u][1] = make_float2(dt * x[u].y, dt * x[u].y);
                    y[u][0] = y[u][1] = make_float2(0.0f, 0.0f);
                }
#pragma unroll
                for (int i = 0; i < NI; i++) {
#pragma unroll
                    for (int u = 0; u < U; u++) {
                        const uint32_t tu = min(tt + u, nt - 1);
                        const float4 b = *reinterpret_cast<const float4*>(Bs + tu * NP + 4 * (s + NS * i));
                        const float4 c = *reinterpret_cast<const float4*>(Cs + tu * NP + 4 * (s + NS * i));
                        const float2 bp[2] = {make_float2(b.x, b.y), make_float2(b.z, b.w)};     // pairs of rows, as they lie in the registers
                        const float2 cp[2] = {make_float2(c.x, c.y), make_float2(c.z, c.w)};
#pragma unroll
                        for (int k = 0; k < 2; k++)
#pragma unroll
                            for (int j = 0; j < 2; j++) {
                                S[i][k][j] = __ffma2_rn(d2[u], S[i][k][j], __fmul2_rn(bp[k], tx[u][j]));
                                y[u][j] = __ffma2_rn(S[i][k][j], cp[k], y[u][j]);
                            }
                    }
                }
                if (a.mode == 1) continue;                 // no read-out on the walk from an empty state
#pragma unroll
                for (int u = 0; u < U; u++) {
                    const float y0 = y[u][0].x + y[u][0].y, y1 = y[u][1].x + y[u][1].y;
                    if (NS >= 2) {
                        float k = (up ? y1 : y0) + __shfl_xor_sync(0xffffffffu, up ? y0 : y1, NS / 2);
#pragma unroll
                        for (uint32_t o = NS / 4; o > 0; o >>= 1) k += __shfl_xor_sync(0xffffffffu, k, o);
                        const uint32_t col = up ? 1u : 0u;
                        if (writer && tt + u < nt && p0 + col < a.P) out[(size_t)(tt + u) * a.H * a.P + col] = fmaf(dsk, up ? x[u].y : x[u].x, k);
                    } else if (tt + u < nt) {
                        if (p0 < a.P) out[(size_t)(tt + u) * a.H * a.P] = fmaf(dsk, x[u].x, y0);
                        if (p0 + 1 < a.P) out[(size_t)(tt + u) * a.H * a.P + 1] = fmaf(dsk, x[u].y, y1);
                    }
                }
            }
        }
    }
    asm volatile("griddepcontrol.launch_dependents;" ::: "memory");
    if (a.mode == 2 && seg + 1 < n_seg) return;            // only the last segment leaves the carried state
    float* to = a.mode == 1 ? a.seg_state + (size_t)seg * slot_elems + my_block : st;
#pragma unroll
    for (int i = 0; i < 16 * RQ; i++) {
        to[(2 * i) * kSsmThreads + tid] = S[i / 4][(i / 2) % 2][i % 2].x;
        to[(2 * i + 1) * kSsmThreads + tid] = S[i / 4][(i / 2) % 2][i % 2].y;
    }
    if (a.mode == 1 && cb == 0 && tid == 0) a.seg_decay[(size_t)seg * a.H + h] = decay_product;
}
// Starting states of the segments: start[0] is the carried state, start[j] = (product of segment j - 1's decays) start[j - 1] + the
// state segment j - 1 reached from empty.  start[j] replaces reached[j - 1] in place; one thread per state element.
__global__ void k_ssm_fold(float* __restrict__ seg_state, const float* __restrict__ seg_decay, const float* __restrict__ state, const float* __restrict__ ctl,
                           uint32_t H, uint32_t head_elems, uint32_t n_seg) {
    pdl_enter();
    const size_t slot_elems = (size_t)H * head_elems, e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (e >= slot_elems) return;
    const uint32_t h = (uint32_t)(e / head_elems);
    float s = state[(size_t)ctl_word(ctl, ZG_CTL_SLOT) * slot_elems + e];
    for (uint32_t j = 0; j + 1 < n_seg; j++) {
        s = fmaf(seg_decay[(size_t)j * H + h], s, seg_state[(size_t)j * slot_elems + e]);
        seg_state[(size_t)j * slot_elems + e] = s;
    }
}
static size_t ssm_state_elems(uint32_t H, uint32_t N, uint32_t P) {
    const uint32_t CPB = kSsmThreads / ssm_slices(N) * 2;
    return (size_t)H * ((P + CPB - 1) / CPB) * 32 * ssm_rq(N) * kSsmThreads;
}
// Segments a step is cut into: a walk is bound by the dependent issue of its warps (a warp uses about a quarter of its scheduler's
// issue slots), one CTA per (head, column block), so a long step of a model with few of those is cut while the GPU still holds
// no more than about three CTAs per SM — beyond that the second walk of every token costs more than the segments gain
// (measured at 1024 tokens: 32 heads 252 -> 115 us, 64 heads 252 -> 211 us with five segments, 128 heads 308 -> 373 us with
// three).  A segment has at least 64 tokens.
static uint32_t ssm_segments(uint32_t T, uint32_t H, uint32_t N, uint32_t P, uint32_t* seg_len) {
    const uint32_t CPB = kSsmThreads / ssm_slices(N) * 2, ctas = H * ((P + CPB - 1) / CPB);
    uint32_t n = 448 / (ctas ? ctas : 1);
    if (n > 8) n = 8;
    if (n > T / 64) n = T / 64;
    if (n < 2) { *seg_len = T; return 1; }
    const uint32_t len = ((T + n - 1) / n + kSsmTile - 1) / kSsmTile * kSsmTile;
    *seg_len = len;
    return (T + len - 1) / len;
}

// ── MIN_GRU, RG_LRU: gated recurrences per channel ───────────────────────────────────────────────────────────────
// S_t = a_t S_{t-1} + b_t is a linear recurrence per channel whose coefficients do not depend on the state, so the step's
// tokens are cut into up to 64 segments that are walked side by side: thread (channel, segment) first walks its segment
// from an empty state, keeping the product of the a_t and the value reached; the segments' (product, value) pairs are then
// folded in order, which gives every segment the state it starts from; the second walk writes the outputs.  A single-token
// step is one segment of one token.  A CELL names the recurrence: what it reads per (token, channel), what it keeps per
// channel, how a token advances (product, state), and what leaves the unit.
constexpr int kGruChannels = 16, kGruMaxSegments = 64;
// minimal gated recurrent unit: z = sigmoid(zl), candidate u + 1/2 (u >= 0) or sigmoid(u), S <- (1 - z) S + z c, out = S silu(g)
struct MinGruCell {
    const float* proj; uint32_t rs, z_off, u_off, g_off;
    struct Chan {};
    struct Raw { float zl, u, gl; };
    __device__ __forceinline__ Chan channel(uint32_t) const { return Chan(); }
    __device__ __forceinline__ Raw load(uint32_t t, uint32_t c, bool out) const {
        const float* row = proj + (size_t)t * rs;
        Raw r; r.zl = row[z_off + c]; r.u = row[u_off + c]; r.gl = out ? row[g_off + c] : 0.0f;
        return r;
    }
    __device__ __forceinline__ void step(const Chan&, const Raw& r, float& A, float& S) const {
        const float z = sigmoidf_(r.zl), cand = r.u >= 0.0f ? r.u + 0.5f : sigmoidf_(r.u);
        A *= 1.0f - z;
        S = fmaf(z, cand, (1.0f - z) * S);
    }
    __device__ __forceinline__ float out(const Raw& r, float S) const { return S * (r.gl * sigmoidf_(r.gl)); }
};
// real-gated linear recurrent unit: r = sigmoid(rl + br), i = sigmoid(il + bi), log a = -c r softplus(lam),
// S <- a S + sqrt(1 - a^2) (i u), out = S act(y).  1 - a^2 = -expm1(2 log a) keeps its digits where a is close to 1.
template <typename WT>
struct RgLruCell {
    const float* u; const float* gates; const float* y; const WT* wts;
    uint32_t u_rs, u_off, g_rs, r_off, i_off, g_bw, g_bs, y_rs, y_off, rb_off, ib_off, lam_off, act;
    float c;
    struct Chan { float br, bi, rate; uint32_t gcol; };
    struct Raw { float rl, il, u, y; };
    __device__ __forceinline__ Chan channel(uint32_t ch) const {
        Chan k; k.br = wld(wts, (size_t)rb_off + ch); k.bi = wld(wts, (size_t)ib_off + ch); k.rate = c * softplusf_(wld(wts, (size_t)lam_off + ch));
        k.gcol = (ch / g_bw) * g_bs + ch % g_bw;
        return k;
    }
    __device__ __forceinline__ Raw load(uint32_t t, uint32_t ch, bool out) const {
        const uint32_t gcol = (ch / g_bw) * g_bs + ch % g_bw;
        const float* g = gates + (size_t)t * g_rs + gcol;
        Raw r; r.rl = g[r_off]; r.il = g[i_off]; r.u = u[(size_t)t * u_rs + u_off + ch]; r.y = out ? y[(size_t)t * y_rs + y_off + ch] : 0.0f;
        return r;
    }
    __device__ __forceinline__ void step(const Chan& k, const Raw& r, float& A, float& S) const {
        const float la = -k.rate * sigmoidf_(r.rl + k.br), a = expf(la);
        A *= a;
        S = fmaf(a, S, sqrtf(-expm1f(2.0f * la)) * (sigmoidf_(r.il + k.bi) * r.u));
    }
    __device__ __forceinline__ float out(const Raw& r, float S) const { return S * seq_epilogue(r.y, act); }
};
template <typename Cell>
__global__ void __launch_bounds__(kGruChannels * kGruMaxSegments) k_channel_scan(Cell cell, float* __restrict__ dst, float* __restrict__ state,
                                                                                 const float* __restrict__ ctl, uint32_t T, uint32_t W, uint32_t drs, uint32_t seg_len) {
    pdl_enter();
    __shared__ float segA[kGruMaxSegments][kGruChannels], segB[kGruMaxSegments][kGruChannels];
    const uint32_t c = blockIdx.x * kGruChannels + threadIdx.x, seg = threadIdx.y, n_seg = blockDim.y;
    const bool on = c < W;
    const uint32_t t_begin = min(T, seg * seg_len), t_end = min(T, t_begin + seg_len);
    float* st = state + (size_t)ctl_word(ctl, ZG_CTL_SLOT) * W;
    const typename Cell::Chan chan = cell.channel(on ? c : 0);
    float S = 0.0f;
    constexpr int U = 8;                                   // tokens whose loads are in flight together
    if (n_seg > 1) {
        float A = 1.0f;
        if (on)
            for (uint32_t t = t_begin; t < t_end; t += U) {
                typename Cell::Raw raw[U];
#pragma unroll
                for (int i = 0; i < U; i++) raw[i] = cell.load(min(t + i, t_end - 1), c, false);
#pragma unroll
                for (int i = 0; i < U; i++)
                    if (t + i < t_end) cell.step(chan, raw[i], A, S);
            }
        segA[seg][threadIdx.x] = A;
        segB[seg][threadIdx.x] = S;
        __syncthreads();
    }
    if (!on) return;
    S = st[c];
    for (uint32_t j = 0; j < seg; j++) S = fmaf(segA[j][threadIdx.x], S, segB[j][threadIdx.x]);
    for (uint32_t t = t_begin; t < t_end; t += U) {
        typename Cell::Raw raw[U];
#pragma unroll
        for (int i = 0; i < U; i++) raw[i] = cell.load(min(t + i, t_end - 1), c, true);
#pragma unroll
        for (int i = 0; i < U; i++) {
            if (t + i < t_end) {
                float A = 1.0f;
                cell.step(chan, raw[i], A, S);
                dst[(size_t)(t + i) * drs + c] = cell.out(raw[i], S);
            }
        }
    }
    if (seg == n_seg - 1) st[c] = S;
}
// segments of a step of T tokens: four tokens or more each, no empty one at the end (the last leaves the state behind)
static uint32_t scan_segments(uint32_t T, uint32_t* seg_len) {
    uint32_t n_seg = (T + 3) / 4;
    if (n_seg > (uint32_t)kGruMaxSegments) n_seg = kGruMaxSegments;
    *seg_len = (T + n_seg - 1) / n_seg;
    return (T + *seg_len - 1) / *seg_len;
}

// ── GATED_NORM: one CTA per (token, group) ───────────────────────────────────────────────────────────────────────
template <typename WT>
__global__ void k_gated_norm(float* dst, const float* src, const float* __restrict__ gate, const WT* __restrict__ w, uint32_t cols, uint32_t groups,
                             uint32_t gate_rs, uint32_t src_rs, uint32_t dst_rs, float eps) {
    pdl_enter();
    __shared__ float sh[32];
    const uint32_t t = blockIdx.x / groups, gi = blockIdx.x % groups, gs = cols / groups, c0 = gi * gs;
    const float* x = src + (size_t)t * src_rs + c0;
    const float* gt = gate + (size_t)t * gate_rs + c0;
    float* out = dst + (size_t)t * dst_rs + c0;
    constexpr int kKeep = 8;                               // values a thread keeps: groups of up to 8 x blockDim are read once, all loads in flight together
    if (gs <= kKeep * blockDim.x) {
        float v[kKeep], z[kKeep], wv[kKeep];
#pragma unroll
        for (int i = 0; i < kKeep; i++) {
            const uint32_t c = threadIdx.x + i * blockDim.x;
            v[i] = c < gs ? x[c] : 0.0f;
            z[i] = c < gs ? gt[c] : 0.0f;
            wv[i] = c < gs ? wld(w, c0 + c) : 0.0f;
        }
        float q = 0.0f;
#pragma unroll
        for (int i = 0; i < kKeep; i++) { v[i] *= z[i] * sigmoidf_(z[i]); q = fmaf(v[i], v[i], q); }
        const float inv = 1.0f / sqrtf(block_sum(q, sh) / (float)gs + eps);
#pragma unroll
        for (int i = 0; i < kKeep; i++) {
            const uint32_t c = threadIdx.x + i * blockDim.x;
            if (c < gs) out[c] = v[i] * inv * wv[i];
        }
        return;
    }
    float q = 0.0f;
    for (uint32_t c = threadIdx.x; c < gs; c += blockDim.x) {
        const float z = gt[c], v = x[c] * (z * sigmoidf_(z));
        q = fmaf(v, v, q);
    }
    const float inv = 1.0f / sqrtf(block_sum(q, sh) / (float)gs + eps);
    for (uint32_t c = threadIdx.x; c < gs; c += blockDim.x) {
        const float z = gt[c], v = x[c] * (z * sigmoidf_(z));
        out[c] = v * inv * wld(w, c0 + c);
    }
}

// ── HEAD_NORM: one warp per (token, head), in place ──────────────────────────────────────────────────────────────
template <typename WT>
__global__ void k_head_norm(float* x, const WT* __restrict__ w, const float* __restrict__ ctl, uint32_t T, uint32_t heads, uint32_t dim, uint32_t rs,
                            uint32_t period, float eps, float coef) {
    pdl_enter();
    const uint32_t item = blockIdx.x * (blockDim.x >> 5) + (threadIdx.x >> 5), lane = threadIdx.x & 31;
    if (item >= T * heads) return;
    const uint32_t t = item / heads, hd = item % heads;
    float* v = x + (size_t)t * rs + (size_t)hd * dim;
    float q = 0.0f;
    for (uint32_t c = lane; c < dim; c += 32) q = fmaf(v[c], v[c], q);
    float mult = 1.0f / sqrtf(warp_sum(q) / (float)dim + eps);
    if (period) {
        const uint32_t pos = (uint32_t)ctl_word(ctl, ZG_CTL_POS) + t;
        mult *= fmaf(coef, logf((float)((pos + 1) / period) + 1.0f), 1.0f);
    }
    for (uint32_t c = lane; c < dim; c += 32) v[c] = v[c] * wld(w, c) * mult;
}

// ── ACTIVATION ───────────────────────────────────────────────────────────────────────────────────────────────────
// four elements per thread (n a multiple of 4, both buffers on 16-byte boundaries) or one
template <bool VEC>
__global__ void k_activation(float* dst, const float* src, uint32_t n, uint32_t kind, float p) {
    pdl_enter();
    const size_t e = (size_t)blockIdx.x * blockDim.x + threadIdx.x;
    if (VEC) {
        if (4 * e >= n) return;
        float4 v = reinterpret_cast<const float4*>(src)[e];
        v.x = seq_activation(v.x, kind, p); v.y = seq_activation(v.y, kind, p); v.z = seq_activation(v.z, kind, p); v.w = seq_activation(v.w, kind, p);
        reinterpret_cast<float4*>(dst)[e] = v;
    } else {
        if (e >= n) return;
        dst[e] = seq_activation(src[e], kind, p);
    }
}

}  // namespace

// shared scratch of a long SSM_SCAN step: per segment but the last, a state (reached, then starting) and the product of its decays per head
size_t zg_rec_op_scratch_elems(const ZgOp& op) {
    if (op.tag != ZG_OP_SSM_SCAN) return 0;
    const ZgSeqOp& s = op.u.seq;
    if (!s.n[1] || !s.n[3] || !s.n[4] || s.n[3] > (uint32_t)kSsmMaxN) return 0;
    uint32_t len;
    const uint32_t n = ssm_segments(s.n[0], s.n[1], s.n[3], s.n[4], &len);
    return n > 1 ? (size_t)(n - 1) * (ssm_state_elems(s.n[1], s.n[3], s.n[4]) + s.n[1]) : 0;
}

// f32 slots per state slot of an op whose state layout is its own (SSM_SCAN); 0 for every other op
extern "C" __attribute__((visibility("default"))) size_t zg_cuda_seq_state_elems(const ZgOp* op) {
    if (!op || op->tag != ZG_OP_SSM_SCAN) return 0;
    const ZgSeqOp& s = op->u.seq;
    if (!s.n[1] || !s.n[3] || !s.n[4] || s.n[3] > (uint32_t)kSsmMaxN) return 0;
    return ssm_state_elems(s.n[1], s.n[3], s.n[4]);
}

bool zg_rec_op_valid(const ZgOp& op, const size_t* elems, size_t n_bufs, char* why, size_t why_n) {
    const ZgSeqOp& s = op.u.seq;
    auto fail = [&](const char* m) { snprintf(why, why_n, "%s", m); return false; };
    auto have = [&](int i) { return s.buf[i] != ZG_NO_BUF && s.buf[i] < n_bufs; };
    auto fits = [&](int i, size_t off, size_t n) { return have(i) && off + n <= elems[s.buf[i]]; };
    auto wfits = [&](int i, uint32_t wdt, size_t off, size_t n) { return wdt <= ZG_W_BF16 && have(i) && (wdt == ZG_W_BF16 ? (off + n + 1) / 2 : off + n) <= elems[s.buf[i]]; };
    switch (op.tag) {
        case ZG_OP_SSM_SCAN: {
            const size_t T = s.n[0], H = s.n[1], G = s.n[2], N = s.n[3], P = s.n[4], xrs = s.n[5], drs = s.n[6];
            if (!T || !H || !G || H % G || !N || N > (size_t)kSsmMaxN || !P) return fail("ssm_scan: shape");
            if (s.off[0] + H * P > xrs || s.off[1] + G * N > xrs || s.off[2] + G * N > xrs || s.off[3] + H > drs) return fail("ssm_scan: columns");
            if (!fits(0, 0, T * H * P) || !fits(1, 0, T * xrs) || !fits(2, 0, T * drs) || !wfits(3, s.n[7], s.off[4], H) || !wfits(3, s.n[7], s.off[5], H) ||
                !wfits(3, s.n[7], s.off[6], H) || !have(4) || elems[s.buf[4]] < ssm_state_elems((uint32_t)H, (uint32_t)N, (uint32_t)P) || !fits(5, 0, ZG_CTL_IDS))
                return fail("ssm_scan: extent");
            if (s.buf[0] == s.buf[1] || s.buf[0] == s.buf[2]) return fail("ssm_scan: in place");
            return true;
        }
        case ZG_OP_MIN_GRU: {
            const size_t T = s.n[0], W = s.n[1], rs = s.n[2], drs = s.n[3];
            if (!T || !W || drs < W || s.off[0] + W > rs || s.off[1] + W > rs || s.off[2] + W > rs) return fail("min_gru: shape");
            if (!fits(0, 0, (T - 1) * drs + W) || !fits(1, 0, T * rs) || !have(2) || elems[s.buf[2]] < W || !fits(3, 0, ZG_CTL_IDS)) return fail("min_gru: extent");
            if (s.buf[0] == s.buf[1]) return fail("min_gru: in place");
            return true;
        }
        case ZG_OP_GATED_NORM: {
            const size_t T = s.n[0], cols = s.n[1], groups = s.n[2], grs = s.n[3], srs = s.n[5], drs = s.n[6];
            if (!T || !cols || !groups || cols % groups || srs < cols || drs < cols || s.off[0] + cols > grs) return fail("gated_norm: shape");
            if (!fits(0, 0, (T - 1) * drs + cols) || !fits(1, 0, (T - 1) * srs + cols) || !fits(2, 0, (T - 1) * grs + s.off[0] + cols) || !wfits(3, s.n[4], s.off[1], cols))
                return fail("gated_norm: extent");
            return true;
        }
        case ZG_OP_HEAD_NORM: {
            const size_t T = s.n[0], heads = s.n[1], dim = s.n[2], rs = s.n[3];
            if (!T || !heads || !dim || s.off[0] + heads * dim > rs) return fail("head_norm: shape");
            if (!fits(0, 0, (T - 1) * rs + s.off[0] + heads * dim) || !wfits(1, s.n[4], s.off[1], dim) || !fits(2, 0, ZG_CTL_IDS)) return fail("head_norm: extent");
            return true;
        }
        case ZG_OP_RG_LRU: {
            const size_t T = s.n[0], W = s.n[1], urs = s.n[2], grs = s.n[3], bw = s.n[4], bs = s.n[5], yrs = s.n[6], drs = s.n[7];
            if (!T || !W || !bw || W % bw || bs < bw || drs < W || s.n[9] > 5 || !(s.f[0] > 0.0f)) return fail("rg_lru: shape");
            const size_t gspan = (W / bw - 1) * bs + bw;
            if (s.off[0] + W > urs || s.off[1] + gspan > grs || s.off[2] + gspan > grs || s.off[3] + W > yrs) return fail("rg_lru: columns");
            if (!fits(0, 0, (T - 1) * drs + W) || !fits(1, 0, (T - 1) * urs + s.off[0] + W) || !fits(2, 0, (T - 1) * grs + (s.off[1] > s.off[2] ? s.off[1] : s.off[2]) + gspan) ||
                !fits(3, 0, (T - 1) * yrs + s.off[3] + W) || !wfits(4, s.n[8], s.off[4], W) || !wfits(4, s.n[8], s.off[5], W) || !wfits(4, s.n[8], s.off[6], W) || !have(5) ||
                elems[s.buf[5]] < W || !fits(6, 0, ZG_CTL_IDS))
                return fail("rg_lru: extent");
            if (s.buf[0] == s.buf[1] || s.buf[0] == s.buf[2] || s.buf[0] == s.buf[3]) return fail("rg_lru: in place");
            return true;
        }
        case ZG_OP_ACTIVATION: {
            if (!s.n[0] || s.n[1] > 4 || (s.n[1] == 4 && !(s.f[0] > 0.0f))) return fail("activation: shape");
            if (!fits(0, 0, s.n[0]) || !fits(1, 0, s.n[0])) return fail("activation: extent");
            return true;
        }
        default: return fail("not a sequence op");
    }
}

uint32_t zg_rec_op_writes(uint32_t tag) {
    switch (tag) {
        case ZG_OP_SSM_SCAN: return 1u | (1u << 4);
        case ZG_OP_MIN_GRU: return 1u | (1u << 2);
        case ZG_OP_RG_LRU: return 1u | (1u << 5);
        default: return 1u;
    }
}

bool zg_launch_rec_op(const ZgOp& op, float* const* bufs, float* scratch, cudaStream_t st) {
    const ZgSeqOp& s = op.u.seq;
    switch (op.tag) {
        case ZG_OP_SSM_SCAN: {
            SsmArgs a;
            a.dst = bufs[s.buf[0]]; a.xbc = bufs[s.buf[1]]; a.dtl = bufs[s.buf[2]]; a.state = bufs[s.buf[4]]; a.ctl = bufs[s.buf[5]];
            a.T = s.n[0]; a.H = s.n[1]; a.G = s.n[2]; a.N = s.n[3]; a.P = s.n[4]; a.x_off = s.off[0]; a.b_off = s.off[1]; a.c_off = s.off[2]; a.dt_off = s.off[3];
            a.xbc_rs = s.n[5]; a.dt_rs = s.n[6];
            const uint32_t NS = ssm_slices(a.N), RQ = ssm_rq(a.N), CPB = kSsmThreads / NS * 2;
            // 16-byte copies when every row of B, C and the CTA's x columns starts on a 16-byte boundary
            a.vec = (a.N % 4 == 0 && a.P % 4 == 0 && a.xbc_rs % 4 == 0 && a.x_off % 4 == 0 && a.b_off % 4 == 0 && a.c_off % 4 == 0 &&
                     (reinterpret_cast<uintptr_t>(a.xbc) & 15) == 0) ? 1u : 0u;
            const size_t smem = ((size_t)2 * kSsmTile * (2 * NS * 16 * RQ + CPB) + 2 * kSsmSpan) * sizeof(float);
            const size_t slot_elems = ssm_state_elems(a.H, a.N, a.P);
            uint32_t seg_len = a.T;
            const uint32_t n_seg = scratch ? ssm_segments(a.T, a.H, a.N, a.P, &seg_len) : 1;
            a.seg_len = seg_len;
            a.seg_state = scratch;
            a.seg_decay = scratch ? scratch + (size_t)(n_seg > 1 ? n_seg - 1 : 0) * slot_elems : nullptr;
#define ZG_SSM(NS_, RQ_)                                                                                                                  \
    ZG_SEQ_WDT(s.n[7], {                                                                                                                  \
        if (smem > 48 * 1024) cudaFuncSetAttribute(k_ssm_scan<WT, NS_, RQ_>, cudaFuncAttributeMaxDynamicSharedMemorySize, (int)smem);     \
        launch_pdl_if(a.T < (uint32_t)kLongWalk, k_ssm_scan<WT, NS_, RQ_>, grid, dim3(kSsmThreads), smem, st, a, wptr<WT>(bufs, s.buf[3], s.off[4]), \
                      wptr<WT>(bufs, s.buf[3], s.off[5]), wptr<WT>(bufs, s.buf[3], s.off[6]));                                            \
    })
#define ZG_SSM_ANY()                                                                                                                      \
    do {                                                                                                                                  \
        if (RQ == 4) ZG_SSM(8, 4);                                                                                                        \
        else if (RQ == 2) ZG_SSM(8, 2);                                                                                                   \
        else switch (NS) {                                                                                                                \
            case 1: ZG_SSM(1, 1); break;                                                                                                  \
            case 2: ZG_SSM(2, 1); break;                                                                                                  \
            case 4: ZG_SSM(4, 1); break;                                                                                                  \
            default: ZG_SSM(8, 1); break;                                                                                                 \
        }                                                                                                                                 \
    } while (0)
            dim3 grid((a.P + CPB - 1) / CPB, a.H, 1);
            if (n_seg > 1) {       // every segment but the last from an empty state, the fold, then every segment from its real start
                a.mode = 1; grid.z = n_seg - 1;
                ZG_SSM_ANY();
                ZG_SEQ_CHECK();
                launch_pdl(k_ssm_fold, dim3((unsigned)((slot_elems + 255) / 256)), dim3(256), 0, st, a.seg_state, (const float*)a.seg_decay, (const float*)a.state, a.ctl, a.H,
                           (uint32_t)(slot_elems / a.H), n_seg);
                ZG_SEQ_CHECK();
                a.mode = 2; grid.z = n_seg;
                ZG_SSM_ANY();
            } else {
                a.mode = 0;
                ZG_SSM_ANY();
            }
#undef ZG_SSM_ANY
#undef ZG_SSM
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_MIN_GRU: {
            const uint32_t T = s.n[0];
            uint32_t seg_len;
            const uint32_t n_seg = scan_segments(T, &seg_len);
            MinGruCell cell;
            cell.proj = bufs[s.buf[1]]; cell.rs = s.n[2]; cell.z_off = s.off[0]; cell.u_off = s.off[1]; cell.g_off = s.off[2];
            launch_pdl_if(T < (uint32_t)kLongWalk, k_channel_scan<MinGruCell>, dim3((s.n[1] + kGruChannels - 1) / kGruChannels), dim3(kGruChannels, n_seg), 0, st, cell, bufs[s.buf[0]], bufs[s.buf[2]],
                          (const float*)bufs[s.buf[3]], T, s.n[1], s.n[3], seg_len);
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_RG_LRU: {
            const uint32_t T = s.n[0];
            uint32_t seg_len;
            const uint32_t n_seg = scan_segments(T, &seg_len);
            ZG_SEQ_WDT(s.n[8], {
                RgLruCell<WT> cell;
                cell.u = bufs[s.buf[1]]; cell.gates = bufs[s.buf[2]]; cell.y = bufs[s.buf[3]]; cell.wts = wptr<WT>(bufs, s.buf[4], 0);
                cell.u_rs = s.n[2]; cell.u_off = s.off[0]; cell.g_rs = s.n[3]; cell.r_off = s.off[1]; cell.i_off = s.off[2]; cell.g_bw = s.n[4]; cell.g_bs = s.n[5];
                cell.y_rs = s.n[6]; cell.y_off = s.off[3]; cell.rb_off = s.off[4]; cell.ib_off = s.off[5]; cell.lam_off = s.off[6]; cell.act = s.n[9]; cell.c = s.f[0];
                launch_pdl_if(T < (uint32_t)kLongWalk, k_channel_scan<RgLruCell<WT>>, dim3((s.n[1] + kGruChannels - 1) / kGruChannels), dim3(kGruChannels, n_seg), 0, st, cell, bufs[s.buf[0]],
                              bufs[s.buf[5]], (const float*)bufs[s.buf[6]], T, s.n[1], s.n[7], seg_len);
            });
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_GATED_NORM: {
            const uint32_t gs = s.n[1] / s.n[2];
            const uint32_t threads = gs <= 64 ? 32 : (gs <= 512 ? 128 : (gs <= 2048 ? 256 : 512));
            ZG_SEQ_WDT(s.n[4], launch_pdl(k_gated_norm<WT>, dim3(s.n[0] * s.n[2]), dim3(threads), 0, st, bufs[s.buf[0]], bufs[s.buf[1]], bufs[s.buf[2]] + s.off[0],
                                          wptr<WT>(bufs, s.buf[3], s.off[1]), s.n[1], s.n[2], s.n[3], s.n[5], s.n[6], s.f[0]));
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_HEAD_NORM: {
            const uint32_t items = s.n[0] * s.n[1];
            ZG_SEQ_WDT(s.n[4], launch_pdl(k_head_norm<WT>, dim3((items + 3) / 4), dim3(128), 0, st, bufs[s.buf[0]] + s.off[0], wptr<WT>(bufs, s.buf[1], s.off[1]), bufs[s.buf[2]], s.n[0], s.n[1],
                                          s.n[2], s.n[3], s.n[5], s.f[0], s.f[1]));
            ZG_SEQ_CHECK();
            return true;
        }
        case ZG_OP_ACTIVATION:
            if (s.n[0] % 4 == 0 && ((reinterpret_cast<uintptr_t>(bufs[s.buf[0]]) | reinterpret_cast<uintptr_t>(bufs[s.buf[1]])) & 15) == 0)
                launch_pdl(k_activation<true>, dim3((s.n[0] / 4 + 255) / 256), dim3(256), 0, st, bufs[s.buf[0]], (const float*)bufs[s.buf[1]], s.n[0], s.n[1], s.f[0]);
            else
                launch_pdl(k_activation<false>, dim3((s.n[0] + 255) / 256), dim3(256), 0, st, bufs[s.buf[0]], (const float*)bufs[s.buf[1]], s.n[0], s.n[1], s.f[0]);
            ZG_SEQ_CHECK();
            return true;
        default:
            zg_set_error("unsupported sequence op tag %u", op.tag);
            return false;
    }
}
